#!/usr/bin/env python
"""Benchmark of the logic-layer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--skip-packed] [--skip-large] [--skip-cpu]
    python bench.py --case NAME [SIZE [NEURONS]]        # one small single-kernel case for a profiler capture

Headline line (one JSON object on stdout, printed by rank 0): the training step of a
784 -> 5 x 16000 -> GroupSum(10, tau=30) logic gate network at batch 128 per GPU (fp32,
random connections, randn weights, Bernoulli(0.19) inputs, uniform labels, CrossEntropy + Adam
lr=0.01), batch-sharded over N GPUs with an exchange of the weight gradients.  The same line carries
  packed_eval   packed-bit inference of the 784 -> 4 x 8000 -> GroupSum(10) network on 2^20 samples (int64
                words), sharded by batch over the N GPUs, checked bit-exactly against the C oracle;
  configs       the wide (9216 -> 4 x 128000, batch 256) and the deep (256 -> 12 x 64000, batch 1024,
                grad_factor 2) training steps and the deep net's packed inference over 2^18 .. 2^24 samples,
                each with its fraction of the measured HBM bandwidth (left out with --skip-large);
  parity        one training step compared with the CPU oracle's step on the concatenated batch of all ranks.

All inputs are synthetic stand-ins with the shapes and value distributions of the data sets the
reference's scripts use (no data set is available offline).

`--impl reference` times the CPU implementation of the same step (the oracle's restatement of the
reference's implementation='python' path, all host threads) on the same global batch and prints a line of
the same shape.
"""
import argparse
import json
import os
import sys
import faulthandler
import gc
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

# name: network widths, classes, tau, batch per GPU, grad_factor, input kind
CONFIGS = {
    "c2": dict(dims=[784] + [16000] * 5, k=10, tau=30.0, batch=128, grad_factor=1.0, p_one=0.19),
    "c4": dict(dims=[9216] + [128000] * 4, k=10, tau=100.0, batch=256, grad_factor=1.0, p_one=None),   # thermometer pixels
    "c5": dict(dims=[256] + [64000] * 12, k=2, tau=20.0, batch=1024, grad_factor=2.0, p_one=0.5),
}
TRAIN_DIMS, TRAIN_K, TRAIN_TAU, TRAIN_BATCH = CONFIGS["c2"]["dims"], 10, 30.0, 128
TRAIN_LR = 0.01
EVAL_DIMS = [784] + [8000] * 4
EVAL_K, EVAL_TAU, EVAL_SAMPLES = 10, 10.0, 1 << 20
P_ONE = 0.19
METRIC = "train step samples/s"
UNIT = "samples/s"
WORKLOAD = ("train step: Flatten -> LogicLayer(784,16000) -> 4 x LogicLayer(16000,16000) -> GroupSum(10, tau=30), "
            "CrossEntropy, Adam lr=0.01")

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from ncu captures of single launches
# (summaries are kept in the profiles folder); None where no capture of that kernel exists.
NCU_TRAFFIC = {
    # training kernels at 16000 x 16000, batch 128: cold-cache captures; inside a step the operands are L2-resident
    "forward": 9.49e6, "backward_w": 17.68e6, "backward_x": 17.04e6,
    # packed eval and group bit-sum: captured at 8000 rows x 4096 words per row and
    # scaled by 4 to the 16384 words of the bench (traffic is proportional to the row length; the part of the
    # output still dirty in L2 at the end of the kernel, ~40 MB, is not)
    "eval_packed": 4 * 262.79e6 + (4 * 262.14e6 - 40.7e6), "groupbitsum": 4 * 272.67e6 + (4 * 10.49e6 - 2.3e6),
}


# ----------------------------------------------------------------------------------------------------------
# helpers
# ----------------------------------------------------------------------------------------------------------

def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while a timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(0.002)

    def __enter__(self):
        if self._nv is not None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._thread = None

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def train_bytes_per_step(dims, batch, k):
    """Algorithmic HBM bytes of one training step: per layer every distinct input read once and every output
    written once (forward X+Y+P+I, backward_w X+Y+I+P, backward_x 2X+Y+P+I+C, not for the first layer), parameter
    work 12 P (softmax 2P+3P, Adam 7P), float GroupSum forward+backward 2 (Y_last + 4 B k)."""
    total = 0
    per_kernel = {}
    for li, (n_in, n_out) in enumerate(zip(dims[:-1], dims[1:])):
        X, Y, P, I = 4 * batch * n_in, 4 * batch * n_out, 64 * n_out, 16 * n_out
        C = 8 * (n_in + 1) + 16 * n_out
        total += (X + Y + P + I) + (X + Y + I + P) + 12 * P
        if li > 0:
            total += 2 * X + Y + P + I + C
            per_kernel = {"forward": X + Y + P + I, "backward_w": X + Y + I + P, "backward_x": 2 * X + Y + P + I + C}
    total += 2 * (4 * batch * dims[-1] + 4 * batch * k)
    return total, per_kernel


def eval_bytes_per_sample(dims, k, fused_tail=False):
    """Packed eval, per sample: each layer reads n_in and writes n_out bits-per-sample (1/8 byte each),
    groupbitsum reads n bits and writes k int32.  With the last layer and the group bit-sum in one kernel the
    last layer's output is neither written nor read back."""
    b = sum((n_in + n_out) / 8.0 for n_in, n_out in zip(dims[:-1], dims[1:]))
    b += dims[-1] / 8.0 + 4 * k
    return b - 2 * dims[-1] / 8.0 if fused_tail else b


def build_gpu_model(dims, k, tau, seed, grad_factor=1.0):
    import difflogic_b200 as D
    torch.manual_seed(seed)          # CPU generator: connections; the weights come from the CUDA generator
    torch.cuda.manual_seed(seed)
    layers = [torch.nn.Flatten()]
    for n_in, n_out in zip(dims[:-1], dims[1:]):
        layers.append(D.LogicLayer(n_in, n_out, device="cuda", grad_factor=grad_factor, connections="random"))
    return torch.nn.Sequential(*layers, D.GroupSum(k, tau))


def synthetic_features(name, batch, generator):
    """[batch, n_in] {0,1} floats with the configuration's value distribution."""
    cfg = CONFIGS[name]
    n_in = cfg["dims"][0]
    if cfg["p_one"] is None:
        # 32 x 32 x 3 uint8 pixels, thermometer-encoded at the thresholds 64, 128, 192 (experiments/main.py:56-59)
        pixels = torch.randint(0, 256, (batch, n_in // 3), generator=generator)
        return torch.cat([(pixels >= t) for t in (64, 128, 192)], dim=1).float()
    return (torch.rand(batch, n_in, generator=generator) < cfg["p_one"]).float()


def event_pair():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def all_reduce_list(values, world, op):
    if world == 1:
        return list(values)
    t = torch.tensor(list(values), dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=op)
    return t.tolist()


def all_max(value, world):
    return all_reduce_list([value], world, dist.ReduceOp.MAX)[0]


def median(values):
    s = sorted(values)
    return s[len(s) // 2]


def barrier(world):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


# ----------------------------------------------------------------------------------------------------------
# training step
# ----------------------------------------------------------------------------------------------------------

def time_kernel(fn, flush, iters=20):
    """(hot, cold) microseconds per launch: `iters` back-to-back launches inside one event pair (inputs stay in L2,
    as they do inside a training step), and single launches each preceded by an untimed L2 flush."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    flush.zero_()                      # keeps the GPU busy while the launches are queued
    s, e = event_pair()
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    hot = s.elapsed_time(e) * 1e3 / iters
    cold = []
    for _ in range(iters):
        flush.zero_()
        s, e = event_pair()
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        cold.append(s.elapsed_time(e) * 1e3)
    cold.sort()
    return hot, cold[len(cold) // 2]


def oracle_parity(model, opt, step, name, rank, world):
    """ONE eager training step on a fixed-seed batch per rank, compared on rank 0 with the CPU oracle's step on the
    concatenated batch of all ranks (experiments/main.py:174-181): the mean of the ranks' losses, the averaged weight
    gradient (read back from Adam's first moments, which after the first step from zero are (1 - beta1) times it) and
    the updated weights.  Must run before any other step of `opt`.  Returns a dict (rank 0) or None."""
    from oracle import logic_oracle as O
    cfg = CONFIGS[name]
    dims, k, tau, batch = cfg["dims"], cfg["k"], cfg["tau"], cfg["batch"]
    logic = [m for m in model if hasattr(m, "indices")]
    start = [l.weights.detach().cpu().clone() for l in logic]
    batches = []
    for r in range(world):
        g = torch.Generator().manual_seed(424200 + r)
        batches.append((synthetic_features(name, batch, g), torch.randint(0, k, (batch,), generator=g)))
    x, y = batches[rank]
    loss = step(x.cuda(), y.cuda())
    torch.cuda.synchronize()
    losses = all_reduce_list([float(loss.item())], world, dist.ReduceOp.SUM)
    m = opt.full_exp_avg()                 # under the peer exchange every rank holds the moments of its slices only
    grads = [(m[off:off + cnt] / 0.1).view_as(p).cpu() for p in opt._params for off, cnt in [opt._slices[p]]]
    after = [l.weights.detach().cpu().clone() for l in logic]
    if rank != 0:
        barrier(world)                     # rank 0 is busy on the CPU for a while: nobody starts the next step without it
        return None
    net = O.OracleNet([w.clone() for w in start], [l.indices[0].cpu() for l in logic], [l.indices[1].cpu() for l in logic], k, tau,
                      cfg["grad_factor"])
    ref_loss, _, ref_grads = net.train_step(torch.cat([b[0] for b in batches]), torch.cat([b[1] for b in batches]), lr=TRAIN_LR)
    out = {"ranks": world, "samples": world * batch, "loss": losses[0] / world, "oracle_loss": float(ref_loss)}
    out["loss_rel_err"] = abs(out["loss"] - out["oracle_loss"]) / abs(out["oracle_loss"])
    out["grad_rel_err"] = max(float((g - r).abs().max() / r.abs().max()) for g, r in zip(grads, ref_grads))
    worst = 0.0
    for w, w0, gr in zip(after, start, ref_grads):
        want = w0 - TRAIN_LR * gr / (gr.abs() + 1e-8)            # first Adam step from zero moments
        sure = gr.abs() > 1e-3 * gr.abs().max()                 # where the sign of the gradient is beyond doubt
        worst = max(worst, float((w - want)[sure].abs().max()) / TRAIN_LR)
    out["update_rel_err"] = worst
    out["ok"] = bool(out["loss_rel_err"] <= 1e-5 and out["grad_rel_err"] <= 1e-4 and worst <= 2e-3)
    out["tolerance"] = "loss 1e-5 relative, gradients 1e-4 of the largest entry per tensor, update 2e-3 of lr"
    barrier(world)
    return out


def replica_checksum(opt, world):
    """True when all ranks hold bit-identical parameters (sum of the parameter words, compared as min == max)."""
    s = float(opt.flat_param.view(torch.int32).to(torch.int64).sum().item())
    lo = all_reduce_list([s], world, dist.ReduceOp.MIN)[0]
    hi = all_reduce_list([s], world, dist.ReduceOp.MAX)[0]
    return lo == hi


_PEER_EXCHANGE = {}


class ExchangeFailed(RuntimeError):
    """A wait of the peer-memory exchange ran out during the bench (raised on every rank alike)."""


def peer_exchange_usable(args, world):
    """Whether this box lets every rank map every other rank's buffers and two trial steps of the headline network get
    through the peer-memory exchange with no wait running out (a short limit, so a box without working peer access
    costs seconds).  Decided once, by all ranks together; when it fails the bench runs on NCCL's all-reduce and says so
    in `implementation.exchange`.  Returns (usable, reason)."""
    if "usable" in _PEER_EXCHANGE:
        return _PEER_EXCHANGE["usable"], _PEER_EXCHANGE["why"]
    from difflogic_b200.losses import CrossEntropyLoss
    from difflogic_b200.optim import ExchangeUnavailable, FlatAdam
    from difflogic_b200.training import TrainStep
    cfg = CONFIGS["c2"]
    why = None
    model = build_gpu_model(cfg["dims"], cfg["k"], cfg["tau"], seed=0, grad_factor=cfg["grad_factor"])
    model.train()
    opt = FlatAdam(model.parameters(), lr=TRAIN_LR)
    try:
        opt.enable_exchange(dist.group.WORLD, buckets=args.exchange_buckets, announce_in_backward=args.announce_in_backward,
                            one_pass_bytes=args.one_pass_bytes, packet_bytes=args.packet_bytes, wait_limit_us=3_000_000,
                            push_in_backward=args.push_in_backward)
    except ExchangeUnavailable as e:      # raised on every rank
        why = str(e)
    if why is None:
        step = TrainStep(model, opt, CrossEntropyLoss(), process_group=dist.group.WORLD, world_size=world)
        g = torch.Generator().manual_seed(77)
        for _ in range(2):
            step(synthetic_features("c2", cfg["batch"], g).cuda(), torch.randint(0, cfg["k"], (cfg["batch"],), generator=g).cuda())
        torch.cuda.synchronize()
        failed = all_max(1.0 if opt.exchange_error() else 0.0, world) > 0
        same = replica_checksum(opt, world)
        if failed or not same:
            why = "trial steps failed (a wait for a peer ran out: %s, replicas identical: %s)" % (failed, same)
        step.close()
    _PEER_EXCHANGE["usable"], _PEER_EXCHANGE["why"] = why is None, why
    return why is None, why


def bench_train(name, args, rank, world, headline):
    from difflogic_b200 import _native
    from difflogic_b200.losses import CrossEntropyLoss
    from difflogic_b200.optim import FlatAdam
    from difflogic_b200.training import TrainStep

    cfg = CONFIGS[name]
    dims, k, tau, batch = cfg["dims"], cfg["k"], cfg["tau"], cfg["batch"]
    dev = torch.device("cuda")
    model = build_gpu_model(dims, k, tau, seed=0, grad_factor=cfg["grad_factor"])   # same seed: identical replicas
    model.train()
    if args.optimizer == "torch":
        opt = torch.optim.Adam(model.parameters(), lr=TRAIN_LR, capturable=True, fused=True)
    else:
        opt = FlatAdam(model.parameters(), lr=TRAIN_LR)
    group = dist.group.WORLD if world > 1 else None
    peer = world > 1 and args.exchange == "peer" and args.optimizer == "flat" and peer_exchange_usable(args, world)[0]
    if peer:
        opt.enable_exchange(group, buckets=args.exchange_buckets, announce_in_backward=args.announce_in_backward,
                            one_pass_bytes=args.one_pass_bytes, packet_bytes=args.packet_bytes,
                            push_in_backward=args.push_in_backward, wait_limit_us=5_000_000)
    loss_fn = torch.nn.CrossEntropyLoss() if args.loss == "torch" else CrossEntropyLoss()
    step = TrainStep(model, opt, loss_fn, process_group=group, world_size=world, buckets=args.buckets)

    parity = None
    if headline and args.optimizer == "flat" and not args.skip_cpu:
        parity = oracle_parity(model, opt, step, name, rank, world)

    # synthetic batches, per-rank seed; a pool in pinned host memory and a copy of it in HBM
    g = torch.Generator().manual_seed(1000 + rank)
    pool = 8 if headline else 2
    hx = torch.stack([synthetic_features(name, batch, g) for _ in range(pool)]).pin_memory()
    hy = torch.randint(0, k, (pool, batch), generator=g).pin_memory()
    dx, dy = hx.to(dev), hy.to(dev)

    before = _native.launch_count()
    step.capture(dx[0], dy[0], warmup=3)
    launches_per_step = (_native.launch_count() - before) // 4   # 3 eager warm-up steps + the captured one
    step.capture_resident([dx[i] for i in range(pool)], [dy[i] for i in range(pool)])   # a graph per resident batch
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    K, W = (args.steps if headline else min(args.steps, 20)), max(args.warmup, 3)
    reps = args.reps if headline else 3
    sampler = ClockSampler(torch.cuda.current_device())

    # ---- device-resident: the batches are already in HBM and every step reads its batch where it is (one captured
    # graph per batch of the pool), the step replayed K times, L2 flushed (untimed) between steps; `reps` repetitions of
    # that loop, each reduced to the max over the ranks, the median repetition is reported
    def give_up_if_the_exchange_failed(where):
        # a wait that ran out (5 s each here) would otherwise be paid for again in every step that follows
        if peer and args.inject_exchange_error and rank == world - 1 and not _PEER_EXCHANGE.get("injected"):
            opt.state_t[0, 2] = 1        # as if a wait of the first bucket had run out on this rank
        _PEER_EXCHANGE["injected"] = True
        if peer and all_max(1.0 if opt.exchange_error() else 0.0, world) > 0:
            sampler.__exit__(None, None, None)
            step.close()
            raise ExchangeFailed("a wait for a peer ran out %s" % where)

    for i in range(W):
        step.replay_resident(i % pool)
    barrier(world)
    give_up_if_the_exchange_failed("in the warm-up steps of %s" % name)
    sampler.__enter__()          # clocks are sampled over both timed loops (device-resident and end to end)
    rep_times = []
    for _ in range(reps):
        pairs = []
        for i in range(K):
            if not args.no_flush:
                flush.zero_()
            else:
                flush[:1 << 20].zero_()  # diagnostic: keeps the launch queue ahead without evicting L2
            if peer:
                opt.rank_barrier()       # the flush does not take equally long on every rank: the timed step starts together
            s, e = event_pair()
            s.record()
            loss = step.replay_resident(i % pool)
            e.record()
            pairs.append((s, e))
        barrier(world)
        rep_times.append(sum(s.elapsed_time(e) for s, e in pairs) * 1e-3)
        give_up_if_the_exchange_failed("in a timed repetition of %s" % name)
    rep_times = all_reduce_list(rep_times, world, dist.ReduceOp.MAX)
    t_dev = median(rep_times)
    final_loss = float(loss.item())
    # time stamps the exchange kernels took on the device during the last timed step (peer exchange only)
    exchange_timing = opt.exchange_timing() if peer else None

    bytes_step, per_kernel = train_bytes_per_step(dims, batch, k)
    peak, peak_kind = measured_peak_gbs()
    out = {
        "value": world * batch * K / t_dev,
        "ms_per_step": t_dev / K * 1e3,
        "repetitions": {"count": reps, "steps_each": K, "ms_per_step_min": min(rep_times) / K * 1e3,
                        "ms_per_step_max": max(rep_times) / K * 1e3},
        "gpu_launches": launches_per_step * K,
        "launches_per_step": launches_per_step,
        "loss": final_loss,
        "step_hbm_frac": (bytes_step / (t_dev / K)) / 1e9 / peak,
        "step_algorithmic_bytes": bytes_step,
        "parity": parity,
    }
    if peer:
        last = max(exchange_timing, key=lambda b: b["done_ns"])
        first = min(exchange_timing, key=lambda b: b["entered_ns"])
        out["exchange_last_step"] = {
            "buckets": len(exchange_timing), "forms": [b_["form"] for b_ in exchange_timing], "first_bucket_entered_to_last_done_ns": last["done_ns"] - first["entered_ns"],
            "last_bucket": {k_: v for k_, v in last.items() if k_ not in ("entered_ns", "done_ns", "stamps_ns")},
            # per bucket (parameter order): entered, all gradients seen, own slice done, all slices seen, done -- ns after
            # the first bucket's entry
            "timeline_ns": [[t - first["entered_ns"] for t in b_["stamps_ns"]] for b_ in exchange_timing]}

    if headline:
        # ---- end to end: pinned host batch -> H2D -> step -> loss read back on the host, every step
        for i in range(W):
            step(hx[i % pool], hy[i % pool]).item()
        barrier(world)
        give_up_if_the_exchange_failed("in the warm-up steps of the end-to-end loop")
        e2e_times = []
        for _ in range(max(3, reps // 2)):
            t_rep = 0.0
            for i in range(K):
                flush.zero_()
                if peer:
                    opt.rank_barrier()   # the ranks leave the synchronize below together
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                step(hx[i % pool], hy[i % pool]).item()
                t_rep += time.perf_counter() - t0
            barrier(world)
            e2e_times.append(t_rep)
        e2e_times = all_reduce_list(e2e_times, world, dist.ReduceOp.MAX)
        t_e2e = median(e2e_times)
        out["e2e"] = {"value": world * batch * K / t_e2e, "unit": UNIT, "ms_per_step": t_e2e / K * 1e3,
                      "h2d_bytes_per_step": hx[0].numel() * 4 + hy[0].numel() * 8, "d2h_bytes_per_step": 4,
                      "repetitions": len(e2e_times), "call": "TrainStep.__call__(x_pinned, y_pinned).item()"}
    sampler.__exit__(None, None, None)
    out["clocks"] = sampler.summary()

    # ---- N > 1: no wait for a peer ran out, and the replicas are still bit-identical
    if world > 1:
        err = bool(opt.exchange_error()) if peer else False
        err = all_max(1.0 if err else 0.0, world) > 0
        out["exchange_error"] = err
        out["replicas_identical"] = replica_checksum(opt, world) if args.optimizer == "flat" else None
        if err or out["replicas_identical"] is False:
            step.close()
            raise ExchangeFailed("the gradient exchange failed (error %s, replicas identical %s)" % (err, out["replicas_identical"]))

    # ---- roofline of the three layer kernels at the hidden-layer shape (rank 0 only)
    if headline and rank == 0 and not args.skip_kernel_timing:
        layer = [m for m in model if hasattr(m, "indices")][2]
        a, b = layer.indices
        n = dims[1]
        x = torch.rand(n, batch, device=dev)
        gy = torch.randn(n, batch, device=dev)
        w = layer.weights.detach().clone()
        y = torch.empty(n, batch, device=dev)
        coef = torch.empty(n, 4, device=dev)
        gw = torch.empty(n, 16, device=dev)
        gx = torch.empty(n, batch, device=dev)
        L, st = _native.lib(), torch.cuda.current_stream().cuda_stream
        kernels = {
            "forward": (5, lambda: L.dl_forward_f32(x.data_ptr(), a.data_ptr(), b.data_ptr(), w.data_ptr(), 0, y.data_ptr(),
                                                    coef.data_ptr(), n, n, batch, 1, st)),
            "backward_w": (5, lambda: L.dl_backward_w_f32(x.data_ptr(), a.data_ptr(), b.data_ptr(), gy.data_ptr(), w.data_ptr(), 0,
                                                          gw.data_ptr(), n, n, batch, 1, st)),
            "backward_x": (4, lambda: L.dl_backward_x_f32(x.data_ptr(), coef.data_ptr(), gy.data_ptr(),
                                                          layer.given_x_indices_of_y_start.data_ptr(), layer._plan.data_ptr(),
                                                          1.0, gx.data_ptr(), n, n, batch, 1, st)),
        }
        rows = {}
        for kname, (count, fn) in kernels.items():
            hot, cold = time_kernel(fn, flush)
            rows[kname] = {"launches_per_step": count, "us_l2_resident": hot, "us_cold_l2": cold, "bytes": per_kernel[kname],
                           "achieved_l2_resident": per_kernel[kname] / hot / 1e3, "achieved_cold_l2": per_kernel[kname] / cold / 1e3,
                           "frac_l2_resident": per_kernel[kname] / hot / 1e3 / peak, "frac_cold_l2": per_kernel[kname] / cold / 1e3 / peak}
        dom = max(rows, key=lambda r: rows[r]["launches_per_step"] * rows[r]["us_l2_resident"])
        r = rows[dom]
        out["roofline"] = {"kernel": dom + "_kernel (16000 x 16000, batch 128)", "bound": "hbm", "achieved": r["achieved_l2_resident"],
                           "peak": peak, "unit": "GB/s", "frac": r["frac_l2_resident"], "peak_kind": peak_kind,
                           "traffic": NCU_TRAFFIC.get(dom), "algorithmic_bytes": r["bytes"], "us_per_launch": r["us_l2_resident"],
                           "operands": "L2-resident",
                           "achieved_cold_l2": r["achieved_cold_l2"], "frac_cold_l2": r["frac_cold_l2"],
                           "note": "achieved / frac: algorithmic bytes over the time of back-to-back launches whose operands are "
                                   "L2-resident, as they are inside the step (a layer's working set is 26 MB, written by the "
                                   "kernel before it): a rate against the HBM peak, not HBM traffic (ncu: `traffic` bytes per "
                                   "launch).  *_cold_l2: the same launch after an L2 flush, everything from HBM."}
        out["roofline_kernels"] = rows
    step.close()   # drops the graph (captured collectives) and leaves the peer exchange before the group goes away
    del step, model, opt
    gc.collect()
    torch.cuda.empty_cache()
    return out


# ----------------------------------------------------------------------------------------------------------
# packed-bit inference
# ----------------------------------------------------------------------------------------------------------

def time_launches(fn, iters=10, warm=2):
    for _ in range(warm):
        fn()
    s, e = event_pair()
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) * 1e3 / iters


def bench_packed(args, rank, world):
    import numpy as np
    import difflogic_b200 as D
    from difflogic_b200 import _native, ops

    dev = torch.device("cuda")
    model = build_gpu_model(EVAL_DIMS, EVAL_K, EVAL_TAU, seed=0)
    model.eval()
    layers = [m for m in model if hasattr(m, "indices")]
    local = EVAL_SAMPLES // world                       # whole 64-bit words per rank
    g = torch.Generator().manual_seed(2000 + rank)
    host_bool = torch.empty(local, EVAL_DIMS[0], dtype=torch.bool).pin_memory()
    chunk = 1 << 16
    for s in range(0, local, chunk):
        host_bool[s:s + chunk] = torch.rand(min(chunk, local - s), EVAL_DIMS[0], generator=g) < P_ONE
    dev_bool = host_bool.to(dev)
    packed = D.PackBitsTensor(dev_bool, bit_count=64)
    words0, pad = packed.t, packed.pad_len
    W = words0.shape[1]
    gates = [l._gate_ids() for l in layers]
    # two ping-pong activation buffers, allocated once (the API call allocates per layer)
    bufs = [torch.empty(EVAL_DIMS[1], W, dtype=torch.int64, device=dev) for _ in range(2)]

    # the plan PackBitsTensor.group_sum runs: all layers but the last one kernel each, then the last layer and the
    # group bit-sum in one kernel when its sizes are in that kernel's range
    fused_tail = D.packbitstensor.FUSED_LAST_LAYER and ops.eval_groupbitsum_applicable(bufs[0], EVAL_DIMS[-1], EVAL_K)

    def run_resident():
        cur = words0
        last = len(layers) - 1
        for i, l in enumerate(layers):
            if i == last and fused_tail:
                return ops.eval_groupbitsum(cur, l.indices[0], l.indices[1], gates[i], pad, EVAL_K)
            cur = ops.eval_packed(cur, l.indices[0], l.indices[1], gates[i], out=bufs[i % 2])
        return ops.groupbitsum(cur, pad, EVAL_K)

    K, Wm = max(args.steps, 50), 3
    for _ in range(Wm):
        counts = run_resident()
    # ---- bit-exact check of what is being timed: the first 2^17 samples of this run's input through the C oracle
    check = None
    if rank == 0 and not args.skip_cpu:
        from oracle import logic_oracle as O
        n_check = min(local, 1 << 17)
        idx_a = [l.indices[0].cpu() for l in layers]
        idx_b = [l.indices[1].cpu() for l in layers]
        gate_ids = [gt.cpu().numpy() for gt in gates]
        ref = O.c_packed_net_counts(host_bool[:n_check].numpy(), idx_a, idx_b, gate_ids, EVAL_K, torch.get_num_threads())
        got = counts[:n_check].cpu().numpy()
        check = {"samples": n_check, "bit_exact": bool(np.array_equal(got, np.asarray(ref))), "against": "C oracle (CompiledLogicNet's arithmetic)"}
        if not check["bit_exact"]:
            raise RuntimeError("bench: packed inference differs from the C oracle")
    barrier(world)
    sampler = ClockSampler(torch.cuda.current_device())
    before = _native.launch_count()
    s, e = event_pair()
    with sampler:
        s.record()
        for _ in range(K):
            counts = run_resident()
        e.record()
        barrier(world)
    launches = _native.launch_count() - before
    t_dev = all_max(s.elapsed_time(e) * 1e-3, world)

    # end to end through the public API: bool matrix in pinned host memory -> class counts on the host
    out_host = torch.empty(local, EVAL_K, dtype=torch.int32).pin_memory()

    def run_e2e():
        with torch.no_grad():
            res = model(D.PackBitsTensor(host_bool.to(dev, non_blocking=True), bit_count=64))
        out_host.copy_(res, non_blocking=True)
        torch.cuda.synchronize()

    run_e2e()
    barrier(world)
    Ke = 10
    t0 = time.perf_counter()
    for _ in range(Ke):
        run_e2e()
    barrier(world)
    t_e2e = all_max(time.perf_counter() - t0, world)

    # per-kernel timing on rank 0 (activations of 1 GB >> L2, so every launch streams from HBM)
    peak, peak_kind = measured_peak_gbs()
    res = {
        "workload": "784 -> 4 x 8000 -> GroupSum(10), eval mode, 2^20 samples in int64 words, sharded by batch",
        "metric": "packed-bit inference samples/s", "unit": UNIT,
        "value": EVAL_SAMPLES * K / t_dev, "ms_per_pass": t_dev / K * 1e3, "passes": K, "samples_per_gpu": local,
        "bytes_per_sample": eval_bytes_per_sample(EVAL_DIMS, EVAL_K, fused_tail),
        "bytes_per_sample_layer_by_layer": eval_bytes_per_sample(EVAL_DIMS, EVAL_K), "fused_last_layer": bool(fused_tail),
        "e2e": {"value": EVAL_SAMPLES * Ke / t_e2e, "unit": UNIT, "h2d_bytes_per_step": host_bool.numel(),
                "d2h_bytes_per_step": out_host.numel() * 4, "iterations": Ke},
        "gpu_launches": launches, "clocks": sampler.summary(),
        "check": check,
    }
    res["hbm_frac"] = res["value"] / world * res["bytes_per_sample"] / 1e9 / peak
    if rank == 0:
        l = layers[1]
        x = bufs[0]
        st = torch.cuda.current_stream().cuda_stream
        L = _native.lib()
        n = EVAL_DIMS[1]
        out_counts = torch.empty(local, EVAL_K, dtype=torch.int32, device=dev)
        kern = {
            "eval_packed": (8 * W * 2 * n, lambda: L.dl_eval_packed(x.data_ptr(), l.indices[0].data_ptr(), l.indices[1].data_ptr(),
                                                                   gates[1].data_ptr(), bufs[1].data_ptr(), n, n, W, 64, st)),
            "groupbitsum": (8 * W * n + 4 * local * EVAL_K, lambda: L.dl_groupbitsum(x.data_ptr(), out_counts.data_ptr(), n, W, pad,
                                                                                     EVAL_K, 64, st)),
            # the step in front of the path: bool [samples, 784] (as the user holds it) -> packed words
            "packbits_batch_major": (local * EVAL_DIMS[0] + 8 * W * EVAL_DIMS[0], lambda: L.dl_packbits_batch_major(
                dev_bool.data_ptr(), words0.data_ptr(), EVAL_DIMS[0], local, 64, st)),
        }
        if fused_tail:
            kern["eval_groupbitsum"] = (8 * W * n + 4 * local * EVAL_K, lambda: L.dl_eval_groupbitsum(
                x.data_ptr(), l.indices[0].data_ptr(), l.indices[1].data_ptr(), gates[1].data_ptr(), out_counts.data_ptr(), n, n, W,
                pad, EVAL_K, 64, st))
        rows = {}
        for name, (nbytes, fn) in kern.items():
            us = time_launches(fn)
            rows[name] = {"us": us, "bytes": nbytes, "achieved": nbytes / us / 1e3, "frac": nbytes / us / 1e3 / peak}
        # thermometer encoding + packing of image-shaped input (3 thresholds on 32 x 32 x 3 uint8 pixels), 2^16 images
        images = 1 << 16
        pixels = torch.randint(0, 256, (images, 3072), dtype=torch.uint8, device=dev)
        us = time_launches(lambda: ops.threshold_packbits_batch_major(pixels, (63, 127, 191), 64))
        nbytes = images * 3072 + 3 * 3072 * (images // 64) * 8
        rows["threshold_packbits_batch_major"] = {"us": us, "bytes": nbytes, "achieved": nbytes / us / 1e3,
                                                  "frac": nbytes / us / 1e3 / peak, "images": images}
        del pixels
        res["roofline"] = {"kernel": "eval_kernel (8000 x 8000, %d int64 words per row)" % W, "bound": "hbm",
                           "achieved": rows["eval_packed"]["achieved"], "peak": peak, "unit": "GB/s",
                           "frac": rows["eval_packed"]["frac"], "peak_kind": peak_kind, "traffic": NCU_TRAFFIC["eval_packed"],
                           "algorithmic_bytes": rows["eval_packed"]["bytes"]}
        res["roofline_kernels"] = rows
    return res


def bench_packed_sweep(args, rank, world, piece=1 << 20, exponents=range(18, 25)):
    """Packed inference of the deep net (256 -> 12 x 64000 -> GroupSum(2)) on 2^18 .. 2^24 samples, sharded by batch over
    the ranks, each rank's share processed in pieces of at most 2^20 samples (two ping-pong activation buffers of
    0.5 GB each): one activation of 2^24 samples would be 134 GB."""
    from difflogic_b200 import ops
    cfg = CONFIGS["c5"]
    dims, k = cfg["dims"], cfg["k"]
    dev = torch.device("cuda")
    model = build_gpu_model(dims, k, cfg["tau"], seed=0, grad_factor=cfg["grad_factor"])
    model.eval()
    layers = [m for m in model if hasattr(m, "indices")]
    gates = [l._gate_ids() for l in layers]
    peak, kind = measured_peak_gbs()
    words_piece = piece // 64
    bufs = [torch.empty(dims[1], words_piece, dtype=torch.int64, device=dev) for _ in range(2)]
    g = torch.Generator(device="cuda").manual_seed(3 + rank)
    # packed input of one piece: every bit set with probability 0.5 (random words)
    x_piece = torch.randint(-2 ** 63, 2 ** 63 - 1, (dims[0], words_piece), dtype=torch.int64, device=dev, generator=g)
    rows = []
    for ex in exponents:
        samples = 1 << ex
        local = samples // world
        pieces = [min(piece, local - s0) for s0 in range(0, local, piece)]

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
        barrier(world)
        reps = max(2, min(8, (1 << 23) // samples))
        s, e = event_pair()
        s.record()
        for _ in range(reps):
            one_pass()
        e.record()
        barrier(world)
        ms = all_max(s.elapsed_time(e), world) / reps
        per_sample = eval_bytes_per_sample(dims, k, fused)
        rows.append({"samples": samples, "samples_per_gpu": local, "pieces_per_gpu": len(pieces), "ms_per_pass": ms,
                     "samples_per_s": samples / ms * 1e3, "bytes_per_sample": per_sample, "fused_last_layer": bool(fused),
                     "hbm_frac": samples / world * per_sample / ms / 1e6 / peak})
    del bufs, x_piece, model
    gc.collect()
    torch.cuda.empty_cache()
    return {"workload": "256 -> 12 x 64000 -> GroupSum(2), eval mode, int64 words, sharded by batch, pieces of <= 2^20 samples",
            "unit": UNIT, "peak_gbs": peak, "peak_kind": kind, "sweep": rows}


# ----------------------------------------------------------------------------------------------------------
# CPU arms
# ----------------------------------------------------------------------------------------------------------

def cpu_train_steps(steps, warmup, global_batch=TRAIN_BATCH, budget_s=None):
    """The reference's CPU training step (implementation='python', device='cpu') as restated by the oracle, all host
    threads.  Returns (seconds, steps_done)."""
    from oracle import logic_oracle as O
    torch.manual_seed(0)
    net = O.OracleNet.build(TRAIN_DIMS, TRAIN_K, TRAIN_TAU)
    g = torch.Generator().manual_seed(1000)
    x = (torch.rand(global_batch, TRAIN_DIMS[0], generator=g) < P_ONE).float()
    y = torch.randint(0, TRAIN_K, (global_batch,), generator=g)
    opt = torch.optim.Adam(net.weights, lr=TRAIN_LR)

    def one():
        loss = torch.nn.functional.cross_entropy(net.forward(x, True), y)
        opt.zero_grad()
        loss.backward()
        opt.step()
        return loss.item()

    for _ in range(warmup):
        one()
    t0 = time.perf_counter()
    done = 0
    for _ in range(steps):
        one()
        done += 1
        if budget_s is not None and time.perf_counter() - t0 > budget_s:
            break
    return time.perf_counter() - t0, done


def cpu_packed_baselines(threads):
    """CPU baselines of the packed inference on this host: (a) the net compiled to straight-line C by CompiledLogicNet
    (gcc -O1, num_bits=64: what the reference's experiments/main.py:353-375 builds) on one core and on `threads`
    cores (the generated function is single-threaded; chunks of the batch run in host threads), (b) the C oracle,
    a table-driven interpreter of the same arithmetic.  Both are checked against each other on the first chunk."""
    import numpy as np
    from concurrent.futures import ThreadPoolExecutor
    import difflogic_b200 as D
    from oracle import logic_oracle as O
    torch.manual_seed(0)
    net = O.OracleNet.build(EVAL_DIMS, EVAL_K, EVAL_TAU)
    gate_ids = net.gate_ids()
    x = (torch.rand(1 << 17, EVAL_DIMS[0], generator=torch.Generator().manual_seed(5)) < P_ONE).numpy()
    out = {}
    # (b) interpreter port
    O.c_packed_net_counts(x[:4096], net.idx_a, net.idx_b, gate_ids, EVAL_K, threads)
    t0 = time.perf_counter()
    ref = np.asarray(O.c_packed_net_counts(x, net.idx_a, net.idx_b, gate_ids, EVAL_K, threads))
    out["interpreter"] = {"value": len(x) / (time.perf_counter() - t0), "cores": threads, "samples": len(x)}
    t0 = time.perf_counter()
    O.c_packed_net_counts(x[:1 << 14], net.idx_a, net.idx_b, gate_ids, EVAL_K, 1)
    out["interpreter_single_core"] = {"value": (1 << 14) / (time.perf_counter() - t0), "cores": 1, "samples": 1 << 14}
    # (a) generated C
    layers = [torch.nn.Flatten()]
    for i, (n_in, n_out) in enumerate(zip(EVAL_DIMS[:-1], EVAL_DIMS[1:])):
        layer = D.LogicLayer(n_in, n_out, device="cpu", implementation="python")
        with torch.no_grad():
            layer.weights.copy_(net.weights[i].detach())
        layer.set_connections(net.idx_a[i], net.idx_b[i])
        layers.append(layer)
    compiled = D.CompiledLogicNet(torch.nn.Sequential(*layers, D.GroupSum(EVAL_K, EVAL_TAU, device="cpu")), num_bits=64)
    t0 = time.perf_counter()
    compiled.compile(opt_level=1, jobs=threads)
    out["compile_s"] = time.perf_counter() - t0
    one = 1 << 14
    got = compiled.forward(x[:one]).numpy()
    if not np.array_equal(got, ref[:one]):
        raise RuntimeError("bench: CompiledLogicNet's C and the C oracle disagree")
    t0 = time.perf_counter()
    compiled.forward(x[:one])
    out["compiled_single_core"] = {"value": one / (time.perf_counter() - t0), "cores": 1, "samples": one}
    per = max(1 << 11, len(x) // max(threads, 1))          # one chunk per host thread
    chunks = [x[s:s + per] for s in range(0, len(x), per)]
    with ThreadPoolExecutor(max_workers=threads) as pool:
        t0 = time.perf_counter()
        list(pool.map(compiled.forward, chunks))          # ctypes releases the interpreter lock during the call
        out["compiled"] = {"value": len(x) / (time.perf_counter() - t0), "cores": min(threads, len(chunks)), "samples": len(x)}
    return out


def train_config(world, exchange=None):
    return {"workload": WORKLOAD, "batch_per_gpu": TRAIN_BATCH, "global_batch": TRAIN_BATCH * world,
            "parallelism": "batch-sharded replicas x%d" % world,
            "l2": "flushed between timed steps (256 MiB memset, untimed; several ranks then meet in a device-side barrier, untimed)"}


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)   # a launcher may have set OMP_NUM_THREADS=1 for its ranks; this arm is rank 0 alone
    world = max(1, args.gpus)
    global_batch = TRAIN_BATCH * world
    # bounded sample: the full step on the global batch, as many of the K steps as fit in about a minute
    t, done = cpu_train_steps(args.steps, max(min(args.warmup, 2), 1), global_batch, budget_s=60.0)
    value = global_batch * done / t
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": done,
        "warmup": max(min(args.warmup, 2), 1), "ms_per_step": t / done * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": train_config(world),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": "%d full training steps on the global batch of %d with torch on %d host threads (oracle "
                                   "restatement of the reference's implementation='python' CPU path)" % (done, global_batch, cores)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------------------
# single-kernel cases for profiler captures
# ----------------------------------------------------------------------------------------------------------

def run_case(argv):
    """python bench.py --case eval|gbs|tail [words [neurons]]        packed eval / group bit-sum (k = 10) / last layer +
                                                                      group bit-sum in one kernel; default 4096 x 8000
       python bench.py --case packbits|thrpack [samples [features]]  bool -> words from the batch-major matrix (default
                                                                      2^18 x 784) / uint8 pixels -> 3 thermometer
                                                                      thresholds -> words (default 2^16 x 3072)
       python bench.py --case fwd|bw|bx|bwadam|head [batch [neurons]] training kernels; default 128 x 16000
    Each case builds a square layer with 'random' connections and launches the kernel three times.  The sizes are
    chosen so that a full-metric capture of one launch finishes in seconds (a few hundred MB on the device)."""
    from difflogic_b200 import ops
    which = argv[0]
    dev = "cuda"
    torch.manual_seed(0)

    def connections(n_in, n_out):
        c = torch.randperm(2 * n_out) % n_in
        c = torch.randperm(n_in)[c].reshape(2, n_out)
        return c[0].to(dev), c[1].to(dev)

    if which in ("eval", "gbs", "tail"):
        words = int(argv[1]) if len(argv) > 1 else 4096
        n = int(argv[2]) if len(argv) > 2 else 8000
        a, b = connections(n, n)
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
    elif which in ("packbits", "thrpack"):
        samples = int(argv[1]) if len(argv) > 1 else (1 << 18 if which == "packbits" else 1 << 16)
        n = int(argv[2]) if len(argv) > 2 else (784 if which == "packbits" else 3072)
        if which == "packbits":
            t = torch.rand(samples, n, device=dev) < 0.19
        else:
            t = torch.randint(0, 256, (samples, n), dtype=torch.uint8, device=dev)
        for _ in range(3):
            if which == "packbits":
                ops.packbits_batch_major(t, 64)
            else:
                ops.threshold_packbits_batch_major(t, (63, 127, 191), 64)
    elif which in ("fwd", "bw", "bx", "bwadam", "head", "fwdhead"):
        batch = int(argv[1]) if len(argv) > 1 else 128
        n = int(argv[2]) if len(argv) > 2 else 16000
        a, b = connections(n, n)
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
            elif which == "fwdhead":
                ops.logic_forward_head(x, a, b, w, target, 10, 30.0)
            elif which == "fwd":
                ops.logic_forward(x, a, b, w, ops.W_LOGITS, True)
            elif which == "bw":
                ops.logic_backward_w(x, a, b, gy, w, ops.W_LOGITS)
            else:
                ops.logic_backward_x(x, coef, gy, start, plan, 1.0)
    else:
        raise SystemExit(run_case.__doc__)
    torch.cuda.synchronize()
    print("done", which)


# ----------------------------------------------------------------------------------------------------------

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--reps", type=int, default=10, help="repetitions of the timed --steps loop; the median is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--loss", default="fused", choices=["fused", "torch"],
                    help="fused: difflogic_b200.losses.CrossEntropyLoss (one kernel each way); torch: torch.nn.CrossEntropyLoss")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="N > 1: peer = gradient exchange + Adam over peer memory, per layer, beside the backward pass; "
                         "nccl = NCCL all-reduce")
    ap.add_argument("--exchange-buckets", type=int, default=None, help="peer exchange: buckets (default: one per layer)")
    ap.add_argument("--announce-in-backward", action="store_true",
                    help="peer exchange: backward_w's last block tells the peers (default: the exchange kernel does)")
    ap.add_argument("--one-pass-bytes", type=int, default=8 << 20,
                    help="peer exchange: one-pass form for the last bucket up to this many bytes over NVLink per rank (0: never)")
    ap.add_argument("--packet-bytes", type=int, default=2 << 20,
                    help="peer exchange: buckets up to this many bytes go as packets with the flags inside the data (0: none)")
    ap.add_argument("--push-in-backward", action="store_true",
                    help="peer exchange: backward_w's epilogue pushes the gradient packets (default: the exchange kernel does)")
    ap.add_argument("--inject-exchange-error", action="store_true",
                    help="N > 1, for testing the fallback: the last rank reports an expired wait after the warm-up steps")
    ap.add_argument("--skip-packed", action="store_true")
    ap.add_argument("--skip-large", action="store_true", help="leave out the wide and deep configurations (`configs`)")
    ap.add_argument("--optimizer", default="flat", choices=["flat", "torch"],
                    help="flat: difflogic_b200.optim.FlatAdam (one kernel); torch: torch.optim.Adam(capturable, fused)")
    ap.add_argument("--skip-cpu", action="store_true", help="no CPU work: no oracle checks, no CPU baselines")
    ap.add_argument("--no-flush", action="store_true", help="diagnostic only: do not flush L2 between the timed steps")
    ap.add_argument("--buckets", type=int, default=2, help="NCCL path: all-reduce pieces of the flat gradient buffer (N > 1)")
    ap.add_argument("--skip-kernel-timing", action="store_true", help="leave out the per-kernel roofline timing")
    ap.add_argument("--case", nargs="+", default=None, help="run one small single-kernel case (for profiler captures) and exit")
    args = ap.parse_args()
    # a run that is stuck (e.g. in a collective) ends itself with a traceback instead of holding the GPUs
    faulthandler.dump_traceback_later(1500, exit=True)

    if args.impl == "reference":
        reference_arm(args)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if args.case:
        import __graft_entry__
        __graft_entry__.build()
        run_case(args.case)
        return
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"   # keep NCCL's version banner out of stdout: one JSON line only
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    assert world == args.gpus or world == 1, "launch with torchrun --nproc-per-node %d" % args.gpus
    cores = os.cpu_count() or 1
    if rank == 0:
        torch.set_num_threads(cores)   # CPU checks and baselines run on rank 0; a launcher may have set OMP_NUM_THREADS=1

    import __graft_entry__
    if rank == 0:
        __graft_entry__.build()
    barrier(world)

    def train_bench(name, headline):
        """bench_train; when the peer-memory exchange fails under it (every rank sees that alike), once more over NCCL's
        all-reduce, and the JSON line says so."""
        try:
            return bench_train(name, args, rank, world, headline)
        except ExchangeFailed as e:
            if _PEER_EXCHANGE.get("usable") is False:
                raise
            _PEER_EXCHANGE["usable"], _PEER_EXCHANGE["why"] = False, str(e)
            if rank == 0:
                print("bench: %s; running %s again with NCCL" % (e, name), file=sys.stderr)
            gc.collect()
            torch.cuda.empty_cache()
            return bench_train(name, args, rank, world, headline)

    train = train_bench("c2", True)
    packed = None if args.skip_packed else bench_packed(args, rank, world)
    large = None
    if not args.skip_large:
        large = {}
        for name in ("c4", "c5"):
            r = train_bench(name, False)
            cfg = CONFIGS[name]
            large[name] = {
                "workload": "train step: %d -> %d x %d -> GroupSum(%d, tau=%g), batch %d per GPU, grad_factor %g, CrossEntropy, Adam" % (
                    cfg["dims"][0], len(cfg["dims"]) - 1, cfg["dims"][1], cfg["k"], cfg["tau"], cfg["batch"], cfg["grad_factor"]),
                "value": r["value"], "unit": UNIT, "ms_per_step": r["ms_per_step"], "hbm_frac": r["step_hbm_frac"],
                "algorithmic_bytes": r["step_algorithmic_bytes"], "launches_per_step": r["launches_per_step"], "loss": r["loss"],
                "repetitions": r["repetitions"], "exchange_last_step": r.get("exchange_last_step"),
                "replicas_identical": r.get("replicas_identical")}
        if not args.skip_packed:
            large["c5_sweep"] = bench_packed_sweep(args, rank, world)

    if rank == 0:
        peer = world > 1 and args.exchange == "peer" and args.optimizer == "flat"
        if peer and not _PEER_EXCHANGE.get("usable", True):
            peer, fell_back = False, " (the peer-memory exchange was not usable here: %s)" % _PEER_EXCHANGE["why"]
        else:
            fell_back = ""
        line = {
            "metric": METRIC, "value": train["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": train["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": train_config(world),
            "implementation": {
                "exchange": "none" if world == 1 else ("one kernel per layer over peer memory (CUDA IPC, plain loads and stores): "
                                                       "average, Adam and the new weights, launched beside the backward pass; "
                                                       "small layers as 8-byte packets that carry their own flag"
                                                       if peer else "NCCL all-reduce" + fell_back),
                "execution": "whole step replayed as one CUDA graph",
                "loss": "CrossEntropy (%s)" % ("difflogic_b200.losses.CrossEntropyLoss" if args.loss == "fused"
                                               else "torch.nn.CrossEntropyLoss"),
                "optimizer": "Adam lr=0.01 (%s)" % ("difflogic_b200.optim.FlatAdam" if args.optimizer == "flat"
                                                    else "torch.optim.Adam capturable fused"),
                "timing": "median of %d repetitions of %d steps, CUDA events per step, max over ranks" % (args.reps, args.steps)},
            "e2e": train["e2e"], "gpu_launches": train["gpu_launches"], "launches_per_step": train["launches_per_step"],
            "repetitions": train["repetitions"],
            "exchange_last_step": train.get("exchange_last_step"), "exchange_error": train.get("exchange_error"),
            "replicas_identical": train.get("replicas_identical"),
            "parity": train["parity"], "parity_checked": bool(train["parity"] and train["parity"]["ok"]),
            "clocks": train["clocks"], "loss": train["loss"],
            "step_algorithmic_bytes": train["step_algorithmic_bytes"], "step_hbm_frac": train["step_hbm_frac"],
            "roofline": train.get("roofline"), "roofline_kernels": train.get("roofline_kernels"),
        }
        if packed is not None:
            line["packed_eval"] = packed
        if large is not None:
            line["configs"] = large
        if not args.skip_cpu and world == 1:
            t, done = cpu_train_steps(5, 1, budget_s=20.0)
            line["cpu_baseline"] = {"value": TRAIN_BATCH * done / t, "unit": UNIT, "cores": cores, "kind": "port",
                                    "sample": "%d training steps of the same net at batch 128 (oracle restatement of the "
                                              "reference's implementation='python' CPU path)" % done}
            if packed is not None:
                b = cpu_packed_baselines(cores)
                packed["cpu_baseline"] = {
                    "value": b["compiled"]["value"], "unit": UNIT, "cores": b["compiled"]["cores"], "kind": "port",
                    "sample": "2^17 samples through the net compiled to straight-line C by CompiledLogicNet (gcc -O1, num_bits=64, "
                              "compiled in %.1f s), one chunk of the batch per host thread" % b["compile_s"],
                    "compiled_single_core": b["compiled_single_core"], "interpreter": b["interpreter"],
                    "interpreter_single_core": b["interpreter_single_core"]}
        if train["parity"] is not None and not train["parity"]["ok"]:
            line["parity_failed"] = True
        print(json.dumps(line))
        if line.get("parity_failed"):
            sys.stdout.flush()
            raise RuntimeError("bench: the training step differs from the oracle: %r" % (train["parity"],))
    barrier(world)
    sys.stdout.flush()
    sys.stderr.flush()
    faulthandler.cancel_dump_traceback_later()
    if world > 1:
        # every rank is past the last collective; leave without tearing NCCL down (its teardown has hung here
        # while CUDA graphs with captured collectives were still referenced)
        os._exit(0)


if __name__ == "__main__":
    main()
