"""The bulk-copy staged training forward (rows of 1 KB and more) against the register-staged kernel and the oracle.
Needs a B200; every test is marked gpu."""
import pytest
import torch

from oracle import logic_oracle as O
from tests.helpers import assert_forward_close, random_layer

pytestmark = pytest.mark.gpu

ops = pytest.importorskip("difflogic_b200.ops")
from difflogic_b200 import _native as N  # noqa: E402

# (n_in, n_out, batch): one chunk, a ragged last tile, several chunks with a 16-byte remainder, many tiles
SHAPES = [(50, 64, 256), (33, 40, 260), (12, 24, 516), (300, 1000, 1024), (64, 17, 4096), (100, 2500, 512)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("mode", ["logits", "probs", "argmax"])
def test_staged_forward_equals_plain_forward_and_oracle(shape, mode, monkeypatch):
    n_in, n_out, batch = shape
    a, b, w = random_layer(n_in, n_out, seed=sum(shape))
    x = torch.rand(batch, n_in, generator=torch.Generator().manual_seed(3))
    if mode == "logits":
        ref, w_in, w_mode = O.layer_forward(x, a, b, w, training=True), w, ops.W_LOGITS
    elif mode == "probs":
        p = torch.softmax(w, -1)
        ref, w_in, w_mode = O.mix_gates(x[:, a], x[:, b], p), p, ops.W_PROBS
    else:
        ref, w_in, w_mode = O.layer_forward(x, a, b, w, training=False), w, ops.W_ARGMAX
    xd = x.t().contiguous().cuda()
    args = (xd, a.cuda(), b.cuda(), w_in.cuda(), w_mode, True)
    with N.tuning(N.TUNE_FORWARD_KERNEL, 2):
        y_staged, c_staged = ops.logic_forward(*args)
    with N.tuning(N.TUNE_FORWARD_KERNEL, 1):
        y_plain, c_plain = ops.logic_forward(*args)
    assert torch.equal(y_staged, y_plain) and torch.equal(c_staged, c_plain)     # same arithmetic, to the bit
    assert_forward_close(y_staged.t().cpu(), ref, "staged forward")
    assert N.lib().dl_async_error() == 0


def test_default_and_plain_agree(monkeypatch):
    """Whatever kernel the library picks by default gives the same numbers as the register kernel."""
    a, b, w = random_layer(64, 96, seed=1)
    for batch in (128, 256):
        x = torch.rand(64, batch, device='cuda')
        y, _ = ops.logic_forward(x, a.cuda(), b.cuda(), w.cuda(), ops.W_LOGITS, True)
        with N.tuning(N.TUNE_FORWARD_KERNEL, 1):
            y2, _ = ops.logic_forward(x, a.cuda(), b.cuda(), w.cuda(), ops.W_LOGITS, True)
        assert torch.equal(y, y2)
