"""End-to-end parity of the Python API on the CUDA path: golden fixtures made by the reference,
the CPU oracle, the reference-named native shim, and the packed-bit pipeline.  Needs a B200."""
import os

import numpy as np
import pytest
import torch

import difflogic_b200 as D
from oracle import logic_oracle as O
from tests.helpers import assert_forward_close, assert_grad_close, build_model, logic_layers

pytestmark = pytest.mark.gpu


def _fixture_net(golden_dir, name):
    g = np.load(os.path.join(golden_dir, name))
    dims = [int(v) for v in g["dims"]]
    L = len(dims) - 1
    ws = [torch.tensor(g["w0_%d" % i]) for i in range(L)]
    aa = [torch.tensor(g["a_%d" % i]) for i in range(L)]
    bb = [torch.tensor(g["b_%d" % i]) for i in range(L)]
    return g, dims, ws, aa, bb


@pytest.mark.parametrize("name", ["small_net.npz", "small_net_gf2.npz"])
def test_small_net_against_reference_fixture(golden_dir, name):
    g, dims, ws, aa, bb = _fixture_net(golden_dir, name)
    k, tau, gf = int(g["k"]), float(g["tau"]), float(g["grad_factor"])
    model = build_model(dims, k, tau, ws, aa, bb, grad_factor=gf)
    x = torch.tensor(g["x"]).cuda()
    y = torch.tensor(g["y"]).cuda()
    L = len(dims) - 1

    model.eval()
    with torch.no_grad():
        ev = model(x)
    assert torch.equal(ev.cpu(), torch.tensor(g["eval_logits"]))  # binary inputs, one gate each: exact

    # packed path == CompiledLogicNet counts of the reference, for every word width
    for bits in (8, 16, 32, 64):
        with torch.no_grad():
            counts = model(D.PackBitsTensor(x.bool(), bit_count=bits))
        assert counts.dtype == torch.int32
        assert np.array_equal(counts.cpu().numpy(), g["compiled_counts_%d" % bits]), bits

    model.train()
    xr = x.clone().requires_grad_(True)
    torch.nn.functional.cross_entropy(model(xr), y).backward()
    assert_grad_close(xr.grad, torch.tensor(g["grad_x"]), "grad wrt input")
    for l in logic_layers(model):
        l.weights.grad = None

    opt = torch.optim.Adam(model.parameters(), lr=0.01)
    logits = model(x)
    loss = torch.nn.functional.cross_entropy(logits, y)
    opt.zero_grad()
    loss.backward()
    assert_forward_close(logits, torch.tensor(g["train_logits"]), "train logits")
    assert abs(loss.item() - float(g["loss"])) <= 1e-5 * abs(float(g["loss"]))
    for i, l in enumerate(logic_layers(model)):
        assert_grad_close(l.weights.grad, torch.tensor(g["grad_%d" % i]), "grad layer %d" % i)
    opt.step()
    for i, l in enumerate(logic_layers(model)):
        # Adam's first step moves every weight by ~lr*sign(grad); compare the update, not the weight
        ref_step = torch.tensor(g["w1_%d" % i]) - torch.tensor(g["w0_%d" % i])
        got_step = l.weights.detach().cpu() - torch.tensor(g["w0_%d" % i])
        big = torch.tensor(g["grad_%d" % i]).abs() > 1e-3 * torch.tensor(g["grad_%d" % i]).abs().max()
        assert torch.allclose(got_step[big], ref_step[big], rtol=1e-3, atol=1e-6)


def test_config1_against_reference_fixture(golden_dir):
    """784 -> 4 x 8000 -> GroupSum(10, tau 10), batch 100, seed 0: the reference's CPU-runnable case."""
    g = np.load(os.path.join(golden_dir, "config1.npz"))
    torch.manual_seed(0)
    dims = [784, 8000, 8000, 8000, 8000]
    net = O.OracleNet.build(dims, 10, 10.0)
    x = (torch.rand(100, 784) < 0.19).float()
    y = torch.randint(0, 10, (100,))
    assert np.array_equal(y.numpy(), g["y"])
    model = build_model(dims, 10, 10.0, net.weights, net.idx_a, net.idx_b)
    xd, yd = x.cuda(), y.cuda()

    model.eval()
    with torch.no_grad():
        assert torch.equal(model(xd).cpu(), torch.tensor(g["eval_logits"]))
        counts = model(D.PackBitsTensor(xd.bool(), bit_count=64))
    assert np.array_equal(counts.cpu().numpy(), g["compiled_counts_64"])
    assert np.array_equal(counts.cpu().numpy(), np.rint(g["eval_logits"] * 10.0).astype(np.int32))

    model.train()
    opt = torch.optim.Adam(model.parameters(), lr=0.01)
    logits = model(xd)
    loss = torch.nn.functional.cross_entropy(logits, yd)
    opt.zero_grad()
    loss.backward()
    assert_forward_close(logits, torch.tensor(g["train_logits"]), "config1 logits")
    assert abs(loss.item() - float(g["loss"])) <= 1e-5 * abs(float(g["loss"]))
    # full gradients against the oracle (which the CPU suite pins to the same fixture)
    _, _, ref_grads = net.train_step(x, y)
    for i, l in enumerate(logic_layers(model)):
        assert_grad_close(l.weights.grad, ref_grads[i], "config1 grad layer %d" % i)
        pos = torch.tensor(g["pos_%d" % i])
        got = l.weights.grad.detach().cpu().reshape(-1)[pos]
        scale = float(g["grad_absmax_%d" % i])
        assert (got - torch.tensor(g["grad_sample_%d" % i])).abs().max().item() <= 1e-4 * scale
    opt.step()
    model.eval()
    with torch.no_grad():
        after = model(xd)
    # discrete outputs after the step: at most a few gates may flip on an arg-max tie-break
    ref_after = torch.tensor(g["eval_logits_after_step"])
    assert (after.cpu() - ref_after).abs().max().item() <= 0.5


def test_deep_net_gradients_not_worse_than_reference_fp32():
    """12 layers with grad_factor 2: the reference's own fp32 gradients of the early layers are
    rounding noise, so the kernels are held to the fp32 reference's own distance from fp64."""
    torch.manual_seed(3)
    dims = [64] + [512] * 8
    net = O.OracleNet.build(dims, 2, 20.0, 2.0)
    x = (torch.rand(96, 64) < 0.5).float()
    y = torch.randint(0, 2, (96,))
    net64 = net.double()
    l64 = torch.nn.functional.cross_entropy(net64.forward(x.double(), True), y)
    l64.backward()
    l32 = torch.nn.functional.cross_entropy(net.forward(x, True), y)
    l32.backward()
    model = build_model(dims, 2, 20.0, net.weights, net.idx_a, net.idx_b, grad_factor=2.0)
    model.train()
    torch.nn.functional.cross_entropy(model(x.cuda()), y.cuda()).backward()
    for i, l in enumerate(logic_layers(model)):
        truth = net64.weights[i].grad
        ref_err = (net.weights[i].grad.double() - truth).abs().max().item()
        got_err = (l.weights.grad.detach().cpu().double() - truth).abs().max().item()
        scale = truth.abs().max().item()
        assert got_err <= max(2.0 * ref_err, 1e-4 * scale), (i, got_err, ref_err, scale)


def test_shim_has_the_reference_native_interface():
    import difflogic_b200.difflogic_cuda as dc
    n_in, n_out, batch = 40, 64, 50
    g = torch.Generator().manual_seed(9)
    a = torch.randint(0, n_in, (n_out,), generator=g)
    b = torch.randint(0, n_in, (n_out,), generator=g)
    b[3] = a[3]
    w = torch.softmax(torch.randn(n_out, 16, generator=g), -1)
    x = torch.rand(batch, n_in, generator=g)
    gy = torch.randn(batch, n_out, generator=g)

    xr = x.clone().requires_grad_(True)
    wr = w.clone().requires_grad_(True)
    ref = O.mix_gates(xr[:, a], xr[:, b], wr)
    ref.backward(gy)
    xd, ad, bd, wd, gyd = x.T.contiguous().cuda(), a.cuda(), b.cuda(), w.cuda(), gy.T.contiguous().cuda()
    assert_forward_close(dc.forward(xd, ad, bd, wd).T, ref, "shim forward")
    assert_grad_close(dc.backward_w(xd, ad, bd, gyd), wr.grad, "shim backward_w")
    start, lst = O.csr_of_connections(a.numpy(), b.numpy(), n_in)
    gx = dc.backward_x(xd, ad, bd, wd, gyd, torch.tensor(start).cuda(), torch.tensor(lst).cuda())
    assert_grad_close(gx.T, xr.grad, "shim backward_x")

    t = torch.rand(n_in, 70, generator=g) < 0.5
    words, pad = dc.tensor_packbits_cuda(t.cuda(), 32)
    ref_words, ref_pad = O.pack_bits(t.numpy(), 32)
    assert pad == ref_pad and np.array_equal(words.cpu().numpy(), ref_words)
    gate = torch.randint(0, 16, (n_out,), generator=g).to(torch.uint8)
    out = dc.eval(words, ad, bd, gate.cuda())
    ref_out = O.eval_packed(ref_words, a.numpy(), b.numpy(), gate.numpy())
    assert np.array_equal(out.cpu().numpy(), ref_out)
    assert np.array_equal(dc.groupbitsum(out, pad, 4).cpu().numpy(), O.group_bit_sum(ref_out, ref_pad, 4))
    with pytest.raises(ValueError):
        dc.groupbitsum(out, pad, 5)
    with pytest.raises(ValueError):
        dc.tensor_packbits_cuda(t.cuda(), 7)

    # the reference-named autograd node on top of it
    from difflogic_b200.difflogic import LogicLayerCudaFunction
    xg = xd.clone().requires_grad_(True)
    wg = wd.clone().requires_grad_(True)
    yy = LogicLayerCudaFunction.apply(xg, ad, bd, wg, torch.tensor(start).cuda(), torch.tensor(lst).cuda())
    yy.backward(gyd)
    assert_grad_close(xg.grad.T, xr.grad, "node grad_x")
    assert_grad_close(wg.grad, wr.grad, "node grad_w")


def test_api_surface_and_layouts():
    torch.manual_seed(0)
    layer = D.LogicLayer(20, 48, grad_factor=1.5)
    assert layer.device == 'cuda' and layer.implementation == 'cuda' and layer.connections == 'random'
    assert layer.weights.shape == (48, 16) and layer.weights.is_cuda
    assert layer.indices[0].dtype == torch.int64 and layer.indices[0].is_cuda
    assert layer.given_x_indices_of_y_start.shape == (21,) and layer.given_x_indices_of_y.shape == (96,)
    assert layer.num_neurons == 48 and layer.num_weights == 48
    assert list(layer.state_dict().keys()) == ['weights']
    assert 'train' in repr(layer)
    x = torch.rand(6, 20, device='cuda')
    y = layer(x)
    assert y.shape == (6, 48) and y.stride() == (1, 6)  # transposed view of the feature-major buffer
    gs = D.GroupSum(4, tau=3.0)
    out = gs(y)
    assert out.shape == (6, 4)
    assert torch.allclose(out, y.reshape(6, 4, 12).sum(-1) / 3.0, rtol=1e-5)
    # generic (batch-major, 3-D) inputs still work
    z = torch.rand(2, 3, 8, device='cuda')
    assert torch.allclose(gs(z), z.reshape(2, 3, 4, 2).sum(-1) / 3.0)

    layer.eval()
    p = D.PackBitsTensor(torch.rand(70, 20, device='cuda') < 0.5)
    assert p.bit_count == 32 and p.t.dtype == torch.int32 and p.t.shape == (20, 3) and p.pad_len == 26
    assert p.flatten() is p
    q = layer(p)
    assert q is p and p.t.shape == (48, 3)  # in place on the caller's object
    assert gs(p).shape == (70, 4) and gs(p).dtype == torch.int32
    layer.train()
    with pytest.raises(AssertionError):
        layer(p)
    with pytest.raises(NotImplementedError):
        D.PackBitsTensor(torch.zeros(4, 4, dtype=torch.bool), device='cpu')
    assert len(repr(D.PackBitsTensor(torch.rand(40, 3, device='cuda') < 0.5, bit_count=8)).split('\n')) == 3


def test_unique_connections_layer_trains():
    torch.manual_seed(1)
    layer = D.LogicLayer(16, 40, connections='unique')
    ref = D.LogicLayer(16, 40, device='cpu', connections='unique')
    ref.set_connections(layer.indices[0].cpu(), layer.indices[1].cpu())
    with torch.no_grad():
        ref.weights.copy_(layer.weights.cpu())
    x = torch.rand(9, 16)
    xa = x.clone().cuda().requires_grad_(True)
    xb = x.clone().requires_grad_(True)
    layer(xa).sum().backward()
    ref(xb).sum().backward()
    assert_grad_close(xa.grad, xb.grad, "unique grad_x")
    assert_grad_close(layer.weights.grad, ref.weights.grad, "unique grad_w")


def test_packed_eval_larger_batch_against_oracle_and_float_path():
    torch.manual_seed(4)
    dims = [100, 640, 640, 320]
    net = O.OracleNet.build(dims, 10, 1.0)
    model = build_model(dims, 10, 1.0, net.weights, net.idx_a, net.idx_b)
    model.eval()
    x = torch.rand(5000, 100) < 0.3
    ref = O.packed_net_counts(x.numpy(), net.idx_a, net.idx_b, net.gate_ids(), 10, 64)
    with torch.no_grad():
        counts = model(D.PackBitsTensor(x.cuda(), bit_count=64))
        fl = model(x.cuda().float())
    assert np.array_equal(counts.cpu().numpy(), ref)
    assert np.array_equal(np.rint(fl.cpu().numpy()).astype(np.int32), ref)


def test_flat_adam_matches_torch_adam():
    """FlatAdam (one kernel over a flat parameter buffer) against torch.optim.Adam over several steps."""
    from difflogic_b200.optim import FlatAdam
    torch.manual_seed(2)
    dims = [40, 96, 96, 60]
    net = O.OracleNet.build(dims, 6, 4.0)
    x = (torch.rand(48, 40) < 0.4).float().cuda()
    y = torch.randint(0, 6, (48,)).cuda()
    m1 = build_model(dims, 6, 4.0, net.weights, net.idx_a, net.idx_b)
    m2 = build_model(dims, 6, 4.0, net.weights, net.idx_a, net.idx_b)
    o1 = torch.optim.Adam(m1.parameters(), lr=0.01)
    o2 = FlatAdam(m2.parameters(), lr=0.01)
    for l in logic_layers(m2):
        assert l.weights.data_ptr() >= o2.flat_param.data_ptr()  # parameters became views of the flat buffer
    for step in range(5):
        for m, o in ((m1, o1), (m2, o2)):
            m.train()
            loss = torch.nn.functional.cross_entropy(m(x), y)
            o.zero_grad()
            loss.backward()
            o.step()
        for l1, l2 in zip(logic_layers(m1), logic_layers(m2)):
            assert l2.weights.grad.data_ptr() == o2.grad_view(l2.weights).data_ptr()  # written in place, not copied
            assert torch.allclose(l1.weights, l2.weights, rtol=1e-5, atol=2e-6), step
    assert int(o2.state_t[0].item()) == 5 and int(o2.state_t[1].item()) == 0


def test_captured_train_step_matches_eager():
    """TrainStep.capture(): the CUDA-graph replay of a step gives the same weights as eager steps."""
    from difflogic_b200.optim import FlatAdam
    from difflogic_b200.training import TrainStep
    torch.manual_seed(6)
    dims = [30, 64, 64]
    net = O.OracleNet.build(dims, 4, 2.0)
    xs = [(torch.rand(32, 30) < 0.5).float().cuda() for _ in range(4)]
    ys = [torch.randint(0, 4, (32,)).cuda() for _ in range(4)]
    models = [build_model(dims, 4, 2.0, net.weights, net.idx_a, net.idx_b) for _ in range(2)]
    steps = [TrainStep(m, FlatAdam(m.parameters(), lr=0.01)) for m in models]
    for m in models:
        m.train()
    steps[1].capture(xs[0], ys[0], warmup=0)
    losses = [[], []]
    for i in range(4):
        for s in (0, 1):
            losses[s].append(float(steps[s](xs[i], ys[i]).item()))
    assert np.allclose(losses[0], losses[1], rtol=1e-5)
    for l0, l1 in zip(logic_layers(models[0]), logic_layers(models[1])):
        assert torch.allclose(l0.weights, l1.weights, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("shape", [(128, 10), (7, 3), (1000, 2), (2500, 17)])
def test_cross_entropy_matches_torch(shape):
    from difflogic_b200.losses import CrossEntropyLoss
    batch, k = shape
    g = torch.Generator().manual_seed(batch + k)
    logits = (torch.randn(batch, k, generator=g) * 3).cuda()
    target = torch.randint(0, k, (batch,), generator=g).cuda()
    a = logits.clone().requires_grad_(True)
    b = logits.clone().requires_grad_(True)
    la = CrossEntropyLoss()(a, target)
    lb = torch.nn.functional.cross_entropy(b, target)
    (la * 1.5).backward()
    (lb * 1.5).backward()
    assert abs(la.item() - lb.item()) <= 1e-5 * abs(lb.item()) + 1e-7
    assert_grad_close(a.grad, b.grad, "cross entropy grad", rtol=1e-5)
    # a view of a feature-major GroupSum output works too
    c = logits.t().contiguous().t().requires_grad_(True)
    assert abs(CrossEntropyLoss()(c, target).item() - lb.item()) <= 1e-5 * abs(lb.item()) + 1e-7


@pytest.mark.parametrize("case", [
    ([100, 640, 640, 320], 10, 64 * 64 * 3, 64),     # 192 words per row, slices of 64 words (512-byte rows)
    ([784, 2000, 2000], 10, 64 * 128 * 3, 128),              # 384 words per row, slices of 128 words
])
def test_network_over_column_slices_equals_the_whole_batch(case):
    """dl_eval_packed_pitched: the first layer reads a column slice of the packed input in place and writes a small
    buffer, the other layers run on small buffers, the counts of a slice land in their rows of the whole result.  This
    is how a batch is processed in pieces without copying the input; the counts must equal the one-piece run."""
    from difflogic_b200 import _native as N, ops
    dims, k, batch, slice_words = case
    torch.manual_seed(sum(dims) + k)
    net = O.OracleNet.build(dims, k, 1.0)
    model = build_model(dims, k, 1.0, net.weights, net.idx_a, net.idx_b)
    model.eval()
    x = torch.rand(batch, dims[0]) < 0.4
    packed = D.PackBitsTensor(x.cuda(), bit_count=64)
    words0, W = packed.t, packed.t.shape[1]
    with torch.no_grad():
        whole = model(D.PackBitsTensor(x.cuda(), bit_count=64))
    layers = logic_layers(model)
    gates = [l._gate_ids() for l in layers]
    lib, st = N.lib(), torch.cuda.current_stream().cuda_stream
    counts = torch.full((batch, k), -1, dtype=torch.int32, device="cuda")
    width = max(dims[1:])
    bufs = [torch.empty(width * slice_words, dtype=torch.int64, device="cuda") for _ in range(2)]
    assert W % slice_words == 0
    for si in range(W // slice_words):
        l = layers[0]
        N.check(lib.dl_eval_packed_pitched(words0.data_ptr() + si * slice_words * 8, W * 8, l.indices[0].data_ptr(),
                                           l.indices[1].data_ptr(), gates[0].data_ptr(), bufs[0].data_ptr(), slice_words * 8,
                                           l.in_dim, l.out_dim, slice_words * 8, st))
        cur = bufs[0][:layers[0].out_dim * slice_words].view(layers[0].out_dim, slice_words)
        for i, l in enumerate(layers[1:], start=1):
            nxt = bufs[i % 2][:l.out_dim * slice_words].view(l.out_dim, slice_words)
            cur = ops.eval_packed(cur, l.indices[0], l.indices[1], gates[i], out=nxt)
        counts[si * slice_words * 64:(si + 1) * slice_words * 64] = ops.groupbitsum(cur, 0, k)
    assert torch.equal(counts, whole)
    # a pitch below the row length, or not a multiple of 16, is refused before anything is launched
    l = layers[0]
    args = (l.indices[0].data_ptr(), l.indices[1].data_ptr(), gates[0].data_ptr(), bufs[0].data_ptr())
    assert lib.dl_eval_packed_pitched(words0.data_ptr(), slice_words * 8 - 16, *args, slice_words * 8, l.in_dim, l.out_dim,
                                      slice_words * 8, st) == N.DL_ERR_INVALID_ARG
    assert lib.dl_eval_packed_pitched(words0.data_ptr(), W * 8 + 8, *args, slice_words * 8, l.in_dim, l.out_dim,
                                      slice_words * 8, st) == N.DL_ERR_INVALID_ARG


def test_packbitstensor_is_lazy_but_keeps_the_in_place_contract():
    torch.manual_seed(0)
    l1, l2 = D.LogicLayer(20, 48), D.LogicLayer(48, 40)
    l1.eval(); l2.eval()
    p = D.PackBitsTensor(torch.rand(70, 20, device='cuda') < 0.5, bit_count=64)
    base = p.t.clone()
    assert l2(l1(p)) is p
    assert p.t.shape == (40, 2)                      # reading .t runs both layers
    from difflogic_b200 import ops
    step1 = ops.eval_packed(base, l1.indices[0], l1.indices[1], l1._gate_ids())
    step2 = ops.eval_packed(step1, l2.indices[0], l2.indices[1], l2._gate_ids())
    assert torch.equal(p.t, step2)
    with pytest.raises(AssertionError):
        l1(p)                                        # 40 rows do not fit a layer with 20 inputs
    # a network too wide for the fused kernel still works (layer by layer)
    wide = D.LogicLayer(20, 20000)
    wide.eval()
    q = D.PackBitsTensor(torch.rand(64, 20, device='cuda') < 0.5, bit_count=64)
    assert D.GroupSum(10)(wide(q)).shape == (64, 10)
