"""The last layer's forward in its class-sum form and the head kernel that finishes it, against the oracle: no
output row is stored, the CTAs of the forward kernel add their rows up per class."""
import pytest
import torch

from oracle import logic_oracle as O
from tests.helpers import assert_forward_close, assert_grad_close, random_layer

pytestmark = pytest.mark.gpu

ops = pytest.importorskip("difflogic_b200.ops")
from difflogic_b200 import _native as N  # noqa: E402


# (n_in, n_out, batch, k): runs of 32 rows at batch 128; classes that are not multiples of the run (a run straddles two
# classes); ragged batches (scalar accesses, fewer lanes per row and longer runs); several batch slabs
CASES = [(784, 16000, 128, 10), (300, 3300, 128, 10), (64, 640, 96, 5), (50, 2600, 37, 2), (40, 4096, 6, 4), (90, 1280, 520, 10)]


@pytest.mark.parametrize("shape", CASES)
def test_forward_head_matches_oracle(shape):
    n_in, n_out, batch, k = shape
    tau = 7.0
    a, b, w = random_layer(n_in, n_out, seed=n_out + batch)
    g = torch.Generator().manual_seed(batch)
    x = torch.rand(batch, n_in, generator=g)
    target = torch.randint(0, k, (batch,), generator=g)
    assert ops.forward_head_applicable(n_out, batch, k)
    wr = w.clone().requires_grad_(True)
    y = O.layer_forward(x, a, b, wr, training=True)
    ref_scores = O.group_sum(y, k, tau)
    ref_loss = torch.nn.functional.cross_entropy(ref_scores, target)
    (grad_scores,) = torch.autograd.grad(ref_loss, ref_scores, retain_graph=True)

    xd = x.t().contiguous().cuda()
    loss, scores, grad_classes, coef = ops.logic_forward_head(xd, a.cuda(), b.cuda(), w.cuda(), target.cuda(), k, tau)
    assert_forward_close(scores.cpu(), ref_scores, "scores")
    assert abs(float(loss) - float(ref_loss)) <= 1e-5 * abs(float(ref_loss))
    assert_grad_close(grad_classes.t().cpu() * tau, grad_scores, "gradient w.r.t. the scores")
    assert torch.equal(coef, ops.logic_coefs(w.cuda(), ops.W_LOGITS))
    # twice in a row: the ticket counter is left at zero
    loss2, scores2, _, _ = ops.logic_forward_head(xd, a.cuda(), b.cuda(), w.cuda(), target.cuda(), k, tau)
    assert torch.equal(loss, loss2) and torch.equal(scores, scores2)


def test_forward_head_refuses_classes_shorter_than_a_run():
    lib = N.lib()
    assert lib.dl_forward_class_sums_run(128) == 32 and lib.dl_forward_class_sums_run(6) == 128
    assert lib.dl_forward_class_sums_rows(16000, 128, 10) == 2 * 500
    assert lib.dl_forward_class_sums_rows(300, 128, 10) == 0           # classes of 30 rows, runs of 32
    assert not ops.forward_head_applicable(300, 128, 10)
    null = None
    assert lib.dl_forward_class_sums_f32(null, null, null, null, 0, null, null, 4, 300, 128, 10, 0, null) == N.DL_ERR_INVALID_ARG
    assert lib.dl_forward_class_sums_f32(null, null, null, null, 0, null, null, 4, 301, 128, 10, 0, null) == N.DL_ERR_NOT_DIVISIBLE
