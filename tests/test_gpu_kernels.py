"""Per-kernel parity of the CUDA path against the CPU oracle, through the C ABI (ctypes).
Needs a B200; every test is marked gpu."""
import numpy as np
import pytest
import torch

from oracle import logic_oracle as O
from tests.helpers import assert_forward_close, assert_grad_close, random_layer

pytestmark = pytest.mark.gpu

ops = pytest.importorskip("difflogic_b200.ops")
from difflogic_b200 import _native as N  # noqa: E402

# (n_in, n_out, batch): ragged sizes (batch not a multiple of 4 / 32 / 128, n_out not of 32), one
# column, one float4, several slabs
SHAPES = [(20, 32, 7), (33, 50, 100), (64, 64, 128), (300, 1000, 128), (50, 70, 1), (16, 40, 260), (8, 5, 4),
          (40, 333, 1024), (12, 24, 516)]


def _dev(t):
    return t.cuda().contiguous()


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("mode", ["logits", "probs", "argmax"])
def test_forward_matches_oracle(shape, mode):
    n_in, n_out, batch = shape
    a, b, w = random_layer(n_in, n_out, seed=sum(shape))
    x = torch.rand(batch, n_in, generator=torch.Generator().manual_seed(3))
    if mode == "logits":
        ref = O.layer_forward(x, a, b, w, training=True)
        w_in, w_mode = w, ops.W_LOGITS
    elif mode == "probs":
        p = torch.softmax(w, -1)
        ref = O.mix_gates(x[:, a], x[:, b], p)
        w_in, w_mode = p, ops.W_PROBS
    else:
        ref = O.layer_forward(x, a, b, w, training=False)
        w_in, w_mode = w, ops.W_ARGMAX
    y, coef = ops.logic_forward(_dev(x.T), _dev(a), _dev(b), _dev(w_in), w_mode, want_coef=True)
    torch.cuda.synchronize()
    assert y.shape == (n_out, batch)
    assert_forward_close(y.T, ref, "forward %s %s" % (mode, shape))
    # the coefficient table reproduces the same layer
    c = coef.cpu()
    A, B = x[:, a], x[:, b]
    assert_forward_close(c[:, 0] + c[:, 1] * A + c[:, 2] * B + c[:, 3] * A * B, ref, "coef")
    assert torch.equal(ops.logic_coefs(_dev(w_in), w_mode).cpu(), c)


def test_forward_on_binary_inputs_in_eval_mode_is_exact():
    n_in, n_out, batch = 64, 200, 96
    a, b, w = random_layer(n_in, n_out, seed=5)
    x = (torch.rand(batch, n_in, generator=torch.Generator().manual_seed(1)) < 0.3).float()
    ref = O.layer_forward(x, a, b, w, training=False)
    y, _ = ops.logic_forward(_dev(x.T), _dev(a), _dev(b), _dev(w), ops.W_ARGMAX)
    assert torch.equal(y.T.cpu(), ref)


@pytest.mark.parametrize("shape", SHAPES)
def test_backward_w_matches_oracle(shape):
    n_in, n_out, batch = shape
    a, b, w = random_layer(n_in, n_out, seed=sum(shape) + 1)
    g = torch.Generator().manual_seed(4)
    x = torch.rand(batch, n_in, generator=g)
    gy = torch.randn(batch, n_out, generator=g)
    p = torch.softmax(w.double(), -1)
    gw_mix, _ = O.layer_backward_closed_form(x.double().T.contiguous(), a, b, p, gy.double().T.contiguous())
    gw_logits = O.softmax_backward(w.double(), gw_mix)

    got_mix = ops.logic_backward_w(_dev(x.T), _dev(a), _dev(b), _dev(gy.T), None, ops.W_PROBS)
    got_logits = ops.logic_backward_w(_dev(x.T), _dev(a), _dev(b), _dev(gy.T), _dev(w), ops.W_LOGITS)
    assert_grad_close(got_mix, gw_mix, "backward_w probs %s" % (shape,))
    assert_grad_close(got_logits, gw_logits, "backward_w logits %s" % (shape,))
    assert float(got_mix[:, 0].abs().max()) == 0.0  # gate 0 is the constant 0

    # and against autograd of the reference formulation in fp32
    wr = w.clone().requires_grad_(True)
    O.layer_forward(x, a, b, wr, training=True).backward(gy)
    assert_grad_close(got_logits, wr.grad, "backward_w vs autograd %s" % (shape,))


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("same_input", [False, True])
def test_backward_x_matches_oracle(shape, same_input):
    n_in, n_out, batch = shape
    a, b, w = random_layer(n_in, n_out, seed=sum(shape) + 2, force_same_input=same_input)
    g = torch.Generator().manual_seed(6)
    x = torch.rand(batch, n_in, generator=g)
    gy = torch.randn(batch, n_out, generator=g)
    xr = x.clone().requires_grad_(True)
    O.layer_forward(xr, a, b, w, training=True).backward(gy)

    da, db = _dev(a), _dev(b)
    start, lst = ops.inverse_index(da, db, n_in)
    ref_start, ref_list = O.csr_of_connections(a.numpy(), b.numpy(), n_in)
    assert np.array_equal(start.cpu().numpy(), ref_start) and np.array_equal(lst.cpu().numpy(), ref_list)
    plan = ops.build_backward_plan(da, db, start, lst)
    xd = _dev(x.T)
    _, coef = ops.logic_forward(xd, da, db, _dev(w), ops.W_LOGITS, want_coef=True)
    for scale in (1.0, 2.0):
        gx = ops.logic_backward_x(xd, coef, _dev(gy.T), start, plan, scale)
        assert_grad_close(gx.T, xr.grad * scale, "backward_x %s scale %g" % (shape, scale))
    _, gx64 = O.layer_backward_closed_form(x.double().T.contiguous(), a, b, torch.softmax(w.double(), -1),
                                           gy.double().T.contiguous())
    assert_grad_close(ops.logic_backward_x(xd, coef, _dev(gy.T), start, plan, 1.0), gx64, "backward_x fp64")


def test_backward_x_with_large_fan_out():
    # 8 inputs feeding 600 neurons: fan-out ~150 per input
    n_in, n_out, batch = 8, 600, 36
    a, b, w = random_layer(n_in, n_out, seed=77)
    g = torch.Generator().manual_seed(8)
    x = torch.rand(batch, n_in, generator=g)
    gy = torch.randn(batch, n_out, generator=g)
    xr = x.clone().requires_grad_(True)
    O.layer_forward(xr, a, b, w, training=True).backward(gy)
    da, db = _dev(a), _dev(b)
    start, lst = ops.inverse_index(da, db, n_in)
    plan = ops.build_backward_plan(da, db, start, lst)
    _, coef = ops.logic_forward(_dev(x.T), da, db, _dev(w), ops.W_LOGITS, want_coef=True)
    gx = ops.logic_backward_x(_dev(x.T), coef, _dev(gy.T), start, plan, 1.0)
    assert_grad_close(gx.T, xr.grad, "fan-out 150")


# ------------------------------------------------------------------------------------------------
# packed path: bit-exact
# ------------------------------------------------------------------------------------------------

PACK_SHAPES = [(5, 1), (7, 8), (20, 37), (33, 64), (16, 100), (784, 129), (12, 1024), (9, 4096 + 17), (130, 640)]


@pytest.mark.parametrize("shape", PACK_SHAPES)
@pytest.mark.parametrize("bits", [8, 16, 32, 64])
def test_packbits_both_layouts(shape, bits):
    n, batch = shape
    t = torch.rand(batch, n, generator=torch.Generator().manual_seed(n + batch)) < 0.4
    ref, ref_pad = O.pack_bits(np.ascontiguousarray(t.numpy().T), bits)
    got, pad = ops.packbits(_dev(t.T), bits)
    assert pad == ref_pad and got.dtype == getattr(torch, "int%d" % bits)
    assert np.array_equal(got.cpu().numpy(), ref)
    got2, pad2 = ops.packbits_batch_major(_dev(t), bits)
    assert pad2 == ref_pad
    assert np.array_equal(got2.cpu().numpy(), ref)


def test_packbits_treats_any_nonzero_byte_as_true():
    t = torch.randint(0, 4, (64, 24), dtype=torch.uint8, generator=torch.Generator().manual_seed(0))
    ref, _ = O.pack_bits(np.ascontiguousarray((t != 0).numpy().T), 64)
    assert np.array_equal(ops.packbits(_dev(t.T), 64)[0].cpu().numpy(), ref)
    assert np.array_equal(ops.packbits_batch_major(_dev(t), 64)[0].cpu().numpy(), ref)


@pytest.mark.parametrize("bits", [8, 16, 32, 64])
@pytest.mark.parametrize("shape", [(20, 32, 1), (33, 50, 3), (64, 100, 16), (100, 333, 70), (8, 5, 257), (50, 37, 300),
                                   (300, 1000, 1024), (40, 16, 2048 + 64), (60, 1003, 130), (16, 2500, 600)])
def test_eval_packed_matches_oracle(bits, shape):
    n_in, n_out, words = shape
    g = torch.Generator().manual_seed(sum(shape) + bits)
    info = torch.iinfo(getattr(torch, "int%d" % bits))
    x = torch.randint(info.min, info.max, (n_in, words), dtype=torch.int64, generator=g).to(getattr(torch, "int%d" % bits))
    a = torch.randint(0, n_in, (n_out,), generator=g)
    b = torch.randint(0, n_in, (n_out,), generator=g)
    gate = (torch.arange(n_out) % 16).to(torch.uint8)[torch.randperm(n_out, generator=g)]
    ref = O.eval_packed(x.numpy(), a.numpy(), b.numpy(), gate.numpy())
    got = ops.eval_packed(_dev(x), _dev(a), _dev(b), _dev(gate))
    assert got.dtype == x.dtype and np.array_equal(got.cpu().numpy(), ref)
    assert N.lib().dl_async_error() == 0  # no bounded wait of the staged kernel ran out


def test_eval_packed_staged_and_plain_kernels_agree(monkeypatch):
    """Rows of 8 KB: the bulk-copy staged kernel is chosen; the switch DL_TUNE_EVAL_KERNEL forces the register kernel."""
    n_in, n_out, words = 500, 777, 1024 + 6
    g = torch.Generator().manual_seed(1)
    x = torch.randint(-2**62, 2**62, (n_in, words), dtype=torch.int64, generator=g)
    a = torch.randint(0, n_in, (n_out,), generator=g)
    b = torch.randint(0, n_in, (n_out,), generator=g)
    gate = torch.randint(0, 16, (n_out,), generator=g).to(torch.uint8)
    ref = O.eval_packed(x.numpy(), a.numpy(), b.numpy(), gate.numpy())
    staged = ops.eval_packed(_dev(x), _dev(a), _dev(b), _dev(gate))
    with N.tuning(N.TUNE_EVAL_KERNEL, 1):
        plain = ops.eval_packed(_dev(x), _dev(a), _dev(b), _dev(gate))
    assert np.array_equal(staged.cpu().numpy(), ref) and np.array_equal(plain.cpu().numpy(), ref)
    assert N.lib().dl_async_error() == 0


def test_argmax_gates_first_maximum_on_ties():
    w = torch.randn(300, 16, generator=torch.Generator().manual_seed(2))
    w[5, 3] = w[5, 9] = 10.0
    w[6] = 0.0
    got = ops.argmax_gates(_dev(w)).cpu()
    assert got.dtype == torch.uint8 and torch.equal(got.long(), w.argmax(-1))
    assert got[5] == 3 and got[6] == 0


@pytest.mark.parametrize("bits", [8, 16, 32, 64])
@pytest.mark.parametrize("case", [(30, 3, 37), (40, 10, 64), (8000, 10, 200), (64, 2, 4096), (12, 1, 130), (6000, 2, 1000),
                                  (50, 50, 77), (130, 10, 128 * 70), (2000, 2, 4160), (4100, 1, 2048)])
def test_groupbitsum_matches_oracle(bits, case):
    n, k, batch = case
    t = torch.rand(n, batch, generator=torch.Generator().manual_seed(n + k + batch)) < 0.5
    words, pad = O.pack_bits(t.numpy(), bits)
    # garbage in the pad bits must not leak into the result (NOT-type gates set them)
    if pad:
        u = words.view(O.BITS_TO_NPU[bits])
        u[:, -1] |= np.array(~((1 << (bits - pad)) - 1) & ((1 << bits) - 1)).astype(O.BITS_TO_NPU[bits])
    ref = O.group_bit_sum(words, pad, k)
    assert np.array_equal(ref, t.numpy().reshape(k, n // k, batch).sum(1).T)
    got = ops.groupbitsum(_dev(torch.from_numpy(words)), pad, k)
    assert got.dtype == torch.int32 and got.shape == (batch, k) and got.is_contiguous()
    assert np.array_equal(got.cpu().numpy(), ref)


def test_groupbitsum_staged_and_plain_kernels_agree(monkeypatch):
    """Rows of 2 KB: the bulk-copy staged kernel is chosen; the switch DL_TUNE_GROUPBITSUM_KERNEL forces the register kernel."""
    n, k, batch = 3000, 10, 16384 - 5
    t = torch.rand(n, batch, generator=torch.Generator().manual_seed(12)) < 0.5
    words, pad = O.pack_bits(t.numpy(), 64)
    ref = O.group_bit_sum(words, pad, k)
    xd = _dev(torch.from_numpy(words))
    staged = ops.groupbitsum(xd, pad, k)
    with N.tuning(N.TUNE_GROUPBITSUM_KERNEL, 1):
        plain = ops.groupbitsum(xd, pad, k)
    assert np.array_equal(staged.cpu().numpy(), ref) and np.array_equal(plain.cpu().numpy(), ref)
    assert N.lib().dl_async_error() == 0


def test_groupbitsum_rejects_indivisible_rows():
    x = torch.zeros(10, 4, dtype=torch.int64, device="cuda")
    with pytest.raises(ValueError):
        ops.groupbitsum(x, 0, 3)


# ------------------------------------------------------------------------------------------------
# float GroupSum
# ------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("case", [(30, 3, 7, 2.0), (16000, 10, 128, 30.0), (8000, 10, 100, 10.0), (64, 2, 1024, 20.0),
                                  (36, 1, 130, 1.0), (1280, 10, 513, 3.0)])
def test_groupsum_forward_backward(case):
    n, k, batch, tau = case
    g = torch.Generator().manual_seed(n + batch)
    x = torch.rand(batch, n, generator=g)
    ref = O.group_sum(x.double(), k, tau)
    for _ in range(2):  # twice: the workspace counters must come back to zero
        got = ops.groupsum(_dev(x.T), k, tau)
        assert_forward_close(got, ref, "groupsum %s" % (case,))
    go = torch.randn(batch, k, generator=g)
    xr = x.clone().requires_grad_(True)
    O.group_sum(xr, k, tau).backward(go)
    gx = ops.groupsum_backward(_dev(go), n, tau)
    assert gx.shape == (n, batch)
    assert_grad_close(gx.T, xr.grad, "groupsum backward", rtol=1e-6)


# ------------------------------------------------------------------------------------------------
# argument checking happens on the host, before any launch
# ------------------------------------------------------------------------------------------------

def test_bad_arguments_raise_like_the_reference():
    x = torch.zeros(4, 8, device="cuda")
    a = torch.zeros(3, dtype=torch.int64, device="cuda")
    w = torch.zeros(3, 16, device="cuda")
    with pytest.raises(RuntimeError):
        ops.logic_forward(x.cpu(), a, a, w)          # CPU tensor
    with pytest.raises(RuntimeError):
        ops.logic_forward(x.t(), a, a, w)            # not contiguous
    with pytest.raises(RuntimeError):
        ops.logic_forward(x.double(), a, a, w)       # dtype
    with pytest.raises(ValueError):
        ops.packbits(torch.zeros(3, 8, dtype=torch.bool, device="cuda"), 12)
    assert ops.logic_forward(x[:, :0].contiguous(), a, a, w)[0].shape == (3, 0)  # empty batch is fine


@pytest.mark.parametrize("bits", [8, 64])
@pytest.mark.parametrize("shape", [(37, 3, 4, 5), (1000, 3, 8, 8), (513, 1, 7, 9)])
def test_thermometer_packing_from_uint8_images(bits, shape):
    """uint8 pixels -> packed thermometer features, against the reference's float encoding followed by packing."""
    import difflogic_b200 as D
    g = torch.Generator().manual_seed(sum(shape))
    img = torch.randint(0, 256, shape, dtype=torch.uint8, generator=g)
    x = img.float() / 255.0
    feats = torch.cat([(x > ((i + 1) / 4)) for i in range(3)], dim=1).reshape(shape[0], -1)   # experiments/main.py:57
    ref, ref_pad = O.pack_bits(np.ascontiguousarray(feats.numpy().T), bits)
    p = D.PackBitsTensor.from_uint8_thresholds(img.cuda(), (63, 127, 191), bit_count=bits)
    assert p.pad_len == ref_pad and p.bit_count == bits
    assert np.array_equal(p.t.cpu().numpy(), ref)


# ------------------------------------------------------------------------------------------------
# index checks (debug aid)
# ------------------------------------------------------------------------------------------------
def test_check_connections_accepts_a_sound_layer_and_names_the_first_violation():
    a, b, _ = random_layer(30, 64, seed=9, force_same_input=True)
    ad, bd = _dev(a), _dev(b)
    start, lst = ops.inverse_index(ad, bd, 30)
    plan = ops.build_backward_plan(ad, bd, start, lst)
    ops.check_connections(ad, bd, 30)
    ops.check_connections(ad, bd, 30, start, lst, plan)
    bad = ad.clone()
    bad[5] = 30                                               # one past the last input row
    with pytest.raises(ValueError, match="outside"):
        ops.check_connections(bad, bd, 30)
    bad_start = start.clone()
    bad_start[7] = bad_start[6] - 1                           # offsets must not decrease
    with pytest.raises(ValueError, match="offsets"):
        ops.check_connections(ad, bd, 30, bad_start, lst, plan)
    bad_list = lst.clone()
    bad_list[3] = 64
    with pytest.raises(ValueError, match="entry outside"):
        ops.check_connections(ad, bd, 30, start, bad_list, plan)
    bad_plan = plan.clone()
    bad_plan[10, 1] = (int(bad_plan[10, 1]) + 1) % 30         # a partner row that is not the neuron's other input
    with pytest.raises(ValueError, match="does not match"):
        ops.check_connections(ad, bd, 30, start, lst, bad_plan)
    bad_plan = plan.clone()
    bad_plan[0, 0] = 2 * 64 + 1                               # a neuron that does not exist: reported, not dereferenced
    with pytest.raises(ValueError, match="out of range"):
        ops.check_connections(ad, bd, 30, start, lst, bad_plan)


@pytest.mark.parametrize("shape", [(128, 784), (1, 7), (33, 65), (100, 32), (3, 4000)])
def test_transpose_equals_torch(shape):
    x = torch.randn(*shape, device="cuda")
    y = ops.transpose(x)
    assert y.is_contiguous() and torch.equal(y, x.t().contiguous())
    # the first layer of a network takes its batch-major input through it: same output as with a pre-transposed input
    import difflogic_b200 as D
    layer = D.LogicLayer(shape[1], max(64, shape[1]), device="cuda", implementation="cuda")
    layer.eval()
    assert torch.equal(layer(x), layer(x.t().contiguous().t()))
