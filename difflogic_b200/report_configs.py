"""Timings of the larger baseline configurations on one GPU, as JSON lines (the headline benchmark is `bench.py`).

    python -m difflogic_b200.report_configs c4         # wide image-shaped training: 9216 -> 4 x 128000, batch 256
    python -m difflogic_b200.report_configs c5         # deep tabular-shaped training: 256 -> 12 x 64000, batch 1024
    python -m difflogic_b200.report_configs c5-sweep   # packed-bit inference of the c5 net, 2^18 .. 2^24 samples

Training: the whole step (forward, loss, backward, Adam) captured in a CUDA graph, inputs resident on the device,
L2 flushed between the timed steps, timed with CUDA events.  Packed inference: int64 words, the batch processed in
pieces of at most 2^20 samples (two ping-pong activation buffers of 8.4 GB each), the last layer fused with the class
count.  `hbm_frac` relates the algorithmic bytes (every distinct input read once, every output written once) to the
measured copy bandwidth in MEASURED_PEAKS.json next to the package, when that file exists, else to 6650 GB/s.
Synthetic inputs with the configurations' shapes and value distributions; random connections and weights.
"""
import json
import os
import sys

import torch

CONFIGS = {
    # name: (dims, k, tau, batch, grad_factor, probability of a one in the input features)
    "c4": ([9216] + [128000] * 4, 10, 100.0, 256, 1.0, None),
    "c5": ([256] + [64000] * 12, 2, 20.0, 1024, 2.0, 0.5),
}


def train_bytes_per_step(dims, batch, k):
    """Algorithmic bytes of one training step: per layer forward X+Y+P+I, backward_w X+Y+I+P, backward_x 2X+Y+P+I+C (not
    for the first layer), parameter work 12 P, float GroupSum forward + backward 2 (Y_last + 4 B k);
    X = 4 B n_in, Y = 4 B n_out, P = 64 n_out, I = 16 n_out, C = 8 (n_in + 1) + 16 n_out."""
    total = 0
    for li, (n_in, n_out) in enumerate(zip(dims[:-1], dims[1:])):
        X, Y, P, I = 4 * batch * n_in, 4 * batch * n_out, 64 * n_out, 16 * n_out
        C = 8 * (n_in + 1) + 16 * n_out
        total += (X + Y + P + I) + (X + Y + I + P) + 12 * P
        if li > 0:
            total += 2 * X + Y + P + I + C
    return total + 2 * (4 * batch * dims[-1] + 4 * batch * k)


def eval_bytes_per_sample(dims, k, fused_tail):
    b = sum((n_in + n_out) / 8.0 for n_in, n_out in zip(dims[:-1], dims[1:])) + dims[-1] / 8.0 + 4 * k
    return b - 2 * dims[-1] / 8.0 if fused_tail else b


def peak_gbs():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, "fallback"


def build_model(dims, k, tau, grad_factor):
    from . import GroupSum, LogicLayer
    torch.manual_seed(0)
    torch.cuda.manual_seed(0)
    layers = [torch.nn.Flatten()]
    for n_in, n_out in zip(dims[:-1], dims[1:]):
        layers.append(LogicLayer(n_in, n_out, device="cuda", grad_factor=grad_factor, connections="random"))
    return torch.nn.Sequential(*layers, GroupSum(k, tau))


def features(name, batch, n_in, p_one, generator):
    if name == "c4":
        # 32 x 32 x 3 uint8 pixels, thermometer-encoded at the thresholds 64, 128, 192
        pixels = torch.randint(0, 256, (batch, n_in // 3), generator=generator)
        return torch.cat([(pixels >= t) for t in (64, 128, 192)], dim=1).float()
    return (torch.rand(batch, n_in, generator=generator) < p_one).float()


def run_training(name, steps=20, warmup=3):
    from .losses import CrossEntropyLoss
    from .optim import FlatAdam
    from .training import TrainStep
    dims, k, tau, batch, grad_factor, p_one = CONFIGS[name]
    dev = torch.device("cuda")
    model = build_model(dims, k, tau, grad_factor)
    model.train()
    step = TrainStep(model, FlatAdam(model.parameters(), lr=0.01), CrossEntropyLoss())
    g = torch.Generator().manual_seed(1)
    x = features(name, batch, dims[0], p_one, g).to(dev)
    y = torch.randint(0, k, (batch,), generator=g).to(dev)
    step.capture(x, y, warmup=warmup)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(warmup):
        step.replay()
    pairs = []
    for _ in range(steps):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        loss = step.replay()
        e.record()
        pairs.append((s, e))
    torch.cuda.synchronize()
    ms = sum(s.elapsed_time(e) for s, e in pairs) / steps
    nbytes = train_bytes_per_step(dims, batch, k)
    peak, kind = peak_gbs()
    step.close()
    return {"config": name, "workload": "train step %s, GroupSum(%d, tau=%g), batch %d, grad_factor %g, CrossEntropy, Adam" % (
                " -> ".join(str(d) for d in (dims[0], "%d x %d" % (len(dims) - 1, dims[1]))), k, tau, batch, grad_factor),
            "ms_per_step": ms, "samples_per_s": batch / ms * 1e3, "algorithmic_bytes": nbytes,
            "achieved_gbs": nbytes / ms / 1e6, "hbm_frac": nbytes / ms / 1e6 / peak, "peak_gbs": peak, "peak_kind": kind,
            "loss": float(loss.item()), "steps": steps}


def run_packed_sweep(name="c5", piece=1 << 20, exponents=range(18, 25)):
    from . import LogicLayer, ops
    dims, k, tau, _, grad_factor, p_one = CONFIGS[name]
    dev = torch.device("cuda")
    model = build_model(dims, k, tau, grad_factor)
    model.eval()
    layers = [m for m in model if isinstance(m, LogicLayer)]
    gates = [l._gate_ids() for l in layers]
    peak, kind = peak_gbs()
    words_piece = piece // 64
    bufs = [torch.empty(dims[1], words_piece, dtype=torch.int64, device=dev) for _ in range(2)]
    g = torch.Generator(device="cuda").manual_seed(3)
    # packed input of one piece: every bit set with probability p_one (random words: p_one = 0.5)
    x_piece = torch.randint(-2 ** 63, 2 ** 63 - 1, (dims[0], words_piece), dtype=torch.int64, device=dev, generator=g)
    out = []
    for ex in exponents:
        samples = 1 << ex
        pieces = [(min(piece, samples - s0)) for s0 in range(0, samples, piece)]

        def one_pass():
            total = None
            for n in pieces:
                w = n // 64
                cur = x_piece[:, :w].contiguous() if w != words_piece else x_piece
                last = len(layers) - 1
                for i, l in enumerate(layers):
                    if i == last and ops.eval_groupbitsum_applicable(cur, l.out_dim, k):
                        total = ops.eval_groupbitsum(cur, l.indices[0], l.indices[1], gates[i], 0, k)
                        break
                    dst = bufs[i % 2][:, :w] if w == words_piece else torch.empty(l.out_dim, w, dtype=torch.int64, device=dev)
                    cur = ops.eval_packed(cur, l.indices[0], l.indices[1], gates[i], out=dst)
                else:
                    total = ops.groupbitsum(cur, 0, k)
            return total

        fused = ops.eval_groupbitsum_applicable(x_piece[:, :pieces[0] // 64].contiguous(), layers[-1].out_dim, k)
        one_pass()
        torch.cuda.synchronize()
        reps = max(1, min(5, (1 << 22) // samples))
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(reps):
            one_pass()
        e.record()
        torch.cuda.synchronize()
        ms = s.elapsed_time(e) / reps
        per_sample = eval_bytes_per_sample(dims, k, fused)
        out.append({"config": name + "-sweep", "samples": samples, "pieces": len(pieces), "ms_per_pass": ms,
                    "samples_per_s": samples / ms * 1e3, "bytes_per_sample": per_sample, "fused_last_layer": bool(fused),
                    "achieved_gbs": samples * per_sample / ms / 1e6, "hbm_frac": samples * per_sample / ms / 1e6 / peak,
                    "peak_gbs": peak, "peak_kind": kind})
    return out


def main(argv):
    which = argv[0] if argv else ""
    if which in ("c4", "c5"):
        print(json.dumps(run_training(which)))
    elif which == "c5-sweep":
        for row in run_packed_sweep():
            print(json.dumps(row), flush=True)
    else:
        raise SystemExit(__doc__)


if __name__ == "__main__":
    main(sys.argv[1:])
