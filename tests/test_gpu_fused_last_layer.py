"""The fused last-layer + group bit-sum kernel (a cluster of CTAs per class and column block) against the oracle
and against the two separate kernels, through the C ABI.  Needs a B200; every test is marked gpu."""
import numpy as np
import pytest
import torch

from oracle import logic_oracle as O
from tests.helpers import build_model

pytestmark = pytest.mark.gpu

ops = pytest.importorskip("difflogic_b200.ops")
import difflogic_b200 as D  # noqa: E402
from difflogic_b200 import _native as N  # noqa: E402


def _case(n_in, n_out, words, bits, seed):
    g = torch.Generator().manual_seed(seed)
    dt = getattr(torch, "int%d" % bits)
    info = torch.iinfo(dt)
    x = torch.randint(info.min, info.max, (n_in, words), dtype=torch.int64, generator=g).to(dt)
    a = torch.randint(0, n_in, (n_out,), generator=g)
    b = torch.randint(0, n_in, (n_out,), generator=g)
    gate = (torch.arange(n_out) % 16).to(torch.uint8)[torch.randperm(n_out, generator=g)]
    return x, a, b, gate


# (n_in, n_out, words, bits, k, pad_len): rows of 560 B .. 10 KB (one ragged and several column blocks), classes of
# 32 .. 2040 gates (clusters of 2, 4 and 8 CTAs; shares that are not multiples of the 8-gate stage), one class, padding;
# the last two have more units than clusters fit on the GPU: several rounds of the persistent clusters, the last one partial
CASES = [(300, 640, 70, 64, 10, 0), (100, 2000, 300, 64, 10, 13), (64, 1500, 256, 64, 1, 63), (50, 640, 128, 64, 20, 1),
         (40, 1010, 512, 8, 10, 7), (77, 999, 200, 32, 3, 31), (500, 8000, 1282, 64, 10, 5), (30, 4080, 66, 64, 2, 0),
         (90, 330, 96, 64, 10, 2), (64, 1640, 1040, 16, 8, 15), (64, 640, 2304, 64, 10, 3), (40, 660, 4100, 64, 11, 9)]


@pytest.mark.parametrize("case", CASES)
def test_fused_last_layer_matches_oracle_and_separate_kernels(case):
    n_in, n_out, words, bits, k, pad_len = case
    x, a, b, gate = _case(n_in, n_out, words, bits, seed=sum(case))
    xd, ad, bd, gd = x.cuda(), a.cuda(), b.cuda(), gate.cuda()
    assert ops.eval_groupbitsum_applicable(xd, n_out, k)
    ref = O.group_bit_sum(O.eval_packed(x.numpy(), a.numpy(), b.numpy(), gate.numpy()), pad_len, k)
    got = ops.eval_groupbitsum(xd, ad, bd, gd, pad_len, k)
    assert got.dtype == torch.int32 and got.shape == ref.shape
    assert np.array_equal(got.cpu().numpy(), ref)
    two = ops.groupbitsum(ops.eval_packed(xd, ad, bd, gd), pad_len, k)
    assert torch.equal(got, two)
    # a second launch reuses the cluster barriers' phases from scratch: same answer
    assert torch.equal(ops.eval_groupbitsum(xd, ad, bd, gd, pad_len, k), got)
    assert N.lib().dl_async_error() == 0


def test_fused_last_layer_range_and_errors():
    x, a, b, gate = _case(64, 640, 64, 64, seed=1)
    xd = x.cuda()
    assert ops.eval_groupbitsum_applicable(xd, 640, 10)
    assert not ops.eval_groupbitsum_applicable(xd, 640, 64)          # 10 gates per class: too few
    assert not ops.eval_groupbitsum_applicable(xd, 641, 10)          # not divisible
    assert not ops.eval_groupbitsum_applicable(xd[:, :32].contiguous(), 640, 10)   # rows of 256 bytes
    assert not ops.eval_groupbitsum_applicable(xd[:, :63].contiguous(), 640, 10)   # rows not a multiple of 16 bytes
    assert not ops.eval_groupbitsum_applicable(xd, 40000, 10)        # 4000 gates per class: over the share limit
    with pytest.raises(ValueError, match="divisible"):
        ops.eval_groupbitsum(xd, a[:639].cuda(), b[:639].cuda(), gate[:639].cuda(), 0, 10)
    with pytest.raises(RuntimeError, match="range"):
        ops.eval_groupbitsum(xd[:, :32].contiguous(), a.cuda(), b.cuda(), gate.cuda(), 0, 10)


def test_model_uses_fused_last_layer_and_matches_layerwise(monkeypatch):
    torch.manual_seed(11)
    dims = [100, 640, 640, 800]
    net = O.OracleNet.build(dims, 10, 1.0)
    model = build_model(dims, 10, 1.0, net.weights, net.idx_a, net.idx_b)
    model.eval()
    x = torch.rand(5100, 100) < 0.3   # 80 words of 64 bits per row, 20 padding bits
    ref = O.packed_net_counts(x.numpy(), net.idx_a, net.idx_b, net.gate_ids(), 10, 64)
    with torch.no_grad():
        model(D.PackBitsTensor(x.cuda(), bit_count=64))   # the layers' arg-max gate ids are cached from here on
        before = N.launch_count()
        fused = model(D.PackBitsTensor(x.cuda(), bit_count=64))
        fused_launches = N.launch_count() - before
        monkeypatch.setattr(D.packbitstensor, "FUSED_LAST_LAYER", False)
        before = N.launch_count()
        layerwise = model(D.PackBitsTensor(x.cuda(), bit_count=64))
        layerwise_launches = N.launch_count() - before
    assert np.array_equal(fused.cpu().numpy(), ref) and torch.equal(fused, layerwise)
    assert fused_launches == layerwise_launches - 1   # pack, two layers, fused tail  vs  pack, three layers, bit-sum
    # the object stays usable: reading .t afterwards still gives the last layer's output
    monkeypatch.setattr(D.packbitstensor, "FUSED_LAST_LAYER", True)
    p = D.PackBitsTensor(x.cuda(), bit_count=64)
    layers = [m for m in model if isinstance(m, D.LogicLayer)]
    with torch.no_grad():
        for layer in layers:
            p = layer(p)
        counts = D.GroupSum(10)(p)
    assert torch.equal(counts, fused)
    assert p.t.shape == (800, 80) and torch.equal(ops.groupbitsum(p.t, p.pad_len, 10), fused)
