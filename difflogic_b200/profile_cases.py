"""Small single-kernel cases for profiler captures.

    python -m difflogic_b200.profile_cases eval   [words  [neurons]]   # packed eval, default 4096 x 8000
    python -m difflogic_b200.profile_cases gbs    [words  [neurons]]   # group bit-sum, k = 10
    python -m difflogic_b200.profile_cases tail   [words  [neurons]]   # last layer + group bit-sum in one kernel, k = 10
    python -m difflogic_b200.profile_cases fwd|bw|bx [batch [neurons]] # training kernels, default 128 x 16000
    python -m difflogic_b200.profile_cases bwadam [batch [neurons]]    # backward_w with the Adam update in its epilogue
    python -m difflogic_b200.profile_cases head   [batch [neurons]]    # GroupSum + cross-entropy + class-row gradients, k = 10

Each case builds a square layer with 'random' connections and launches the kernel three times.  The sizes are
chosen so that a full-metric capture of one launch finishes in seconds (a few hundred MB on the device).
"""
import sys

import torch

from . import ops


def _connections(n_in, n_out, dev):
    c = torch.randperm(2 * n_out) % n_in
    c = torch.randperm(n_in)[c].reshape(2, n_out)
    return c[0].to(dev), c[1].to(dev)


def main(argv):
    which = argv[0]
    dev = "cuda"
    torch.manual_seed(0)
    if which in ("eval", "gbs", "tail"):
        words = int(argv[1]) if len(argv) > 1 else 4096
        n = int(argv[2]) if len(argv) > 2 else 8000
        a, b = _connections(n, n, dev)
        gate = torch.randint(0, 16, (n,), dtype=torch.uint8, device=dev)
        x = torch.randint(-2 ** 62, 2 ** 62, (n, words), dtype=torch.int64, device=dev)
        out = torch.empty_like(x)
        for _ in range(3):
            if which == "eval":
                ops.eval_packed(x, a, b, gate, out=out)
            elif which == "tail":
                ops.eval_groupbitsum(x, a, b, gate, 0, 10)
            else:
                ops.groupbitsum(x, 0, 10)
    elif which in ("fwd", "bw", "bx", "bwadam", "head"):
        batch = int(argv[1]) if len(argv) > 1 else 128
        n = int(argv[2]) if len(argv) > 2 else 16000
        a, b = _connections(n, n, dev)
        w = torch.randn(n, 16, device=dev)
        x = torch.rand(n, batch, device=dev)
        gy = torch.randn(n, batch, device=dev)
        start, lst = ops.inverse_index(a, b, n)
        plan = ops.build_backward_plan(a, b, start, lst)
        _, coef = ops.logic_forward(x, a, b, w, ops.W_LOGITS, True)
        m1 = torch.zeros(n * 16, device=dev)
        m2 = torch.zeros(n * 16, device=dev)
        state = torch.zeros(2, dtype=torch.int32, device=dev)
        target = torch.randint(0, 10, (batch,), device=dev)
        torch.cuda.synchronize()
        for _ in range(3):
            if which == "bwadam":
                ops.logic_backward_w_adam(x, a, b, gy, w, m1, m2, state, lr=0.01, beta1=0.9, beta2=0.999, eps=1e-8)
            elif which == "head":
                ops.groupsum_cross_entropy(x, target, 10, 30.0)
            elif which == "fwd":
                ops.logic_forward(x, a, b, w, ops.W_LOGITS, True)
            elif which == "bw":
                ops.logic_backward_w(x, a, b, gy, w, ops.W_LOGITS)
            else:
                ops.logic_backward_x(x, coef, gy, start, plan, 1.0)
    else:
        raise SystemExit(__doc__)
    torch.cuda.synchronize()
    print("done", which)


if __name__ == "__main__":
    main(sys.argv[1:])
