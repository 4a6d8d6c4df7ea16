#!/usr/bin/env python
"""Benchmark of the logic-layer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--skip-packed]

Headline line (one JSON object on stdout, printed by rank 0): the training step of a
784 -> 5 x 16000 -> GroupSum(10, tau=30) logic gate network at batch 128 per GPU (fp32,
random connections, randn weights, Bernoulli(0.19) inputs, uniform labels, CrossEntropy + Adam
lr=0.01), batch-sharded over N GPUs with an all-reduce of the weight gradients.  The same line
carries, under "packed_eval", the packed-bit inference of the 784 -> 4 x 8000 -> GroupSum(10)
network on 2^20 samples (int64 words), sharded by batch over the N GPUs.

All inputs are synthetic stand-ins with the shapes and value distributions of the data sets the
reference's scripts use (no data set is available offline).

`--impl reference` times the CPU implementation of the same step (the oracle's restatement of the
reference's implementation='python' path, all host threads) and prints a line of the same shape.
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

TRAIN_DIMS = [784] + [16000] * 5
TRAIN_K, TRAIN_TAU, TRAIN_BATCH, TRAIN_LR = 10, 30.0, 128, 0.01
EVAL_DIMS = [784] + [8000] * 4
EVAL_K, EVAL_TAU, EVAL_SAMPLES = 10, 10.0, 1 << 20
P_ONE = 0.19
METRIC = "train step samples/s"
UNIT = "samples/s"

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


def build_gpu_model(dims, k, tau, seed):
    import difflogic_b200 as D
    torch.manual_seed(seed)          # CPU generator: connections; the weights come from the CUDA generator
    torch.cuda.manual_seed(seed)
    layers = [torch.nn.Flatten()]
    for n_in, n_out in zip(dims[:-1], dims[1:]):
        layers.append(D.LogicLayer(n_in, n_out, device="cuda", connections="random"))
    return torch.nn.Sequential(*layers, D.GroupSum(k, tau))


def event_pair():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def all_max(value, world):
    if world == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def all_sum(value, world):
    if world == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def barrier(world):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


# ----------------------------------------------------------------------------------------------------------
# training step (headline)
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


def bench_train(args, rank, world):
    from difflogic_b200 import _native, ops
    from difflogic_b200.training import TrainStep

    dev = torch.device("cuda")
    model = build_gpu_model(TRAIN_DIMS, TRAIN_K, TRAIN_TAU, seed=0)   # same seed: identical replicas
    model.train()
    if args.optimizer == "torch":
        opt = torch.optim.Adam(model.parameters(), lr=TRAIN_LR, capturable=True, fused=True)
    else:
        from difflogic_b200.optim import FlatAdam
        opt = FlatAdam(model.parameters(), lr=TRAIN_LR)
    group = dist.group.WORLD if world > 1 else None
    if world > 1 and args.exchange == "peer" and args.optimizer == "flat":
        opt.enable_exchange(group)
    if args.loss == "torch":
        loss_fn = torch.nn.CrossEntropyLoss()
    else:
        from difflogic_b200.losses import CrossEntropyLoss
        loss_fn = CrossEntropyLoss()
    step = TrainStep(model, opt, loss_fn, process_group=group, world_size=world, buckets=args.buckets)

    # synthetic batches, per-rank seed; a pool in pinned host memory and a copy of it in HBM
    g = torch.Generator().manual_seed(1000 + rank)
    pool = 8
    hx = (torch.rand(pool, TRAIN_BATCH, TRAIN_DIMS[0], generator=g) < P_ONE).float().pin_memory()
    hy = torch.randint(0, TRAIN_K, (pool, TRAIN_BATCH), generator=g).pin_memory()
    dx, dy = hx.to(dev), hy.to(dev)

    before = _native.launch_count()
    step.capture(dx[0], dy[0], warmup=3)
    launches_per_step = (_native.launch_count() - before) // 4   # 3 eager warm-up steps + the captured one
    sx, sy = step.static_inputs
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    K, W = args.steps, max(args.warmup, 3)
    sampler = ClockSampler(torch.cuda.current_device())

    # ---- device-resident: inputs already in HBM, the step replayed K times, L2 flushed (untimed) between steps
    for i in range(W):
        sx.copy_(dx[i % pool]); sy.copy_(dy[i % pool])
        step.replay()
    barrier(world)
    pairs = []
    sampler.__enter__()          # clocks are sampled over both timed loops (device-resident and end to end)
    for i in range(K):
        if not args.no_flush:
            flush.zero_()
        else:
            flush[:1 << 20].zero_()  # diagnostic: keeps the launch queue ahead without evicting L2
        s, e = event_pair()
        s.record()
        sx.copy_(dx[i % pool], non_blocking=True)
        sy.copy_(dy[i % pool], non_blocking=True)
        loss = step.replay()
        e.record()
        pairs.append((s, e))
    barrier(world)
    t_dev = sum(s.elapsed_time(e) for s, e in pairs) * 1e-3
    t_dev = all_max(t_dev, world)
    final_loss = float(loss.item())
    # time stamps the exchange kernel took on the device during the last timed step (peer exchange only)
    exchange_timing = opt.exchange_timing() if getattr(opt, "exchange_enabled", False) else None

    # ---- end to end: pinned host batch -> H2D -> step -> loss read back on the host, every step
    for i in range(W):
        step(hx[i % pool], hy[i % pool]).item()
    barrier(world)
    t_e2e = 0.0
    for i in range(K):
        flush.zero_()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        step(hx[i % pool], hy[i % pool]).item()
        t_e2e += time.perf_counter() - t0
    barrier(world)
    sampler.__exit__(None, None, None)
    t_e2e = all_max(t_e2e, world)

    bytes_step, per_kernel = train_bytes_per_step(TRAIN_DIMS, TRAIN_BATCH, TRAIN_K)
    peak, peak_kind = measured_peak_gbs()
    out = {
        "value": world * TRAIN_BATCH * K / t_dev,
        "ms_per_step": t_dev / K * 1e3,
        "e2e": {"value": world * TRAIN_BATCH * K / t_e2e, "unit": UNIT, "ms_per_step": t_e2e / K * 1e3,
                "h2d_bytes_per_step": hx[0].numel() * 4 + hy[0].numel() * 8, "d2h_bytes_per_step": 4},
        "gpu_launches": launches_per_step * K,
        "launches_per_step": launches_per_step,
        "exchange_kernel_last_step": exchange_timing,
        "loss": final_loss,
        "step_hbm_frac": (bytes_step / (t_dev / K)) / 1e9 / peak,
        "step_algorithmic_bytes": bytes_step,
        "clocks": sampler.summary(),
    }

    # ---- roofline of the three layer kernels at the hidden-layer shape (rank 0 only)
    if rank == 0 and not args.skip_kernel_timing:
        layer = [m for m in model if hasattr(m, "indices")][2]
        a, b = layer.indices
        n = TRAIN_DIMS[1]
        x = torch.rand(n, TRAIN_BATCH, device=dev)
        gy = torch.randn(n, TRAIN_BATCH, device=dev)
        w = layer.weights.detach()
        y = torch.empty(n, TRAIN_BATCH, device=dev)
        coef = torch.empty(n, 4, device=dev)
        gw = torch.empty(n, 16, device=dev)
        gx = torch.empty(n, TRAIN_BATCH, device=dev)
        L, st = _native.lib(), torch.cuda.current_stream().cuda_stream
        kernels = {
            "forward": (5, lambda: L.dl_forward_f32(x.data_ptr(), a.data_ptr(), b.data_ptr(), w.data_ptr(), 0, y.data_ptr(),
                                                    coef.data_ptr(), n, n, TRAIN_BATCH, 1, st)),
            "backward_w": (5, lambda: L.dl_backward_w_f32(x.data_ptr(), a.data_ptr(), b.data_ptr(), gy.data_ptr(), w.data_ptr(), 0,
                                                          gw.data_ptr(), n, n, TRAIN_BATCH, 1, st)),
            "backward_x": (4, lambda: L.dl_backward_x_f32(x.data_ptr(), coef.data_ptr(), gy.data_ptr(),
                                                          layer.given_x_indices_of_y_start.data_ptr(), layer._plan.data_ptr(),
                                                          1.0, gx.data_ptr(), n, n, TRAIN_BATCH, 1, st)),
        }
        rows = {}
        for name, (count, fn) in kernels.items():
            hot, cold = time_kernel(fn, flush)
            rows[name] = {"launches_per_step": count, "us_hot": hot, "us_cold": cold, "bytes": per_kernel[name],
                          "achieved": per_kernel[name] / hot / 1e3, "achieved_cold": per_kernel[name] / cold / 1e3}
        dom = max(rows, key=lambda r: rows[r]["launches_per_step"] * rows[r]["us_hot"])
        r = rows[dom]
        out["roofline"] = {"kernel": dom + "_kernel (16000 x 16000, batch 128)", "bound": "hbm", "achieved": r["achieved"],
                           "peak": peak, "unit": "GB/s", "frac": r["achieved"] / peak, "peak_kind": peak_kind,
                           "traffic": NCU_TRAFFIC.get(dom), "algorithmic_bytes": r["bytes"], "us_per_launch": r["us_hot"],
                           "achieved_cold_l2": r["achieved_cold"], "frac_cold_l2": r["achieved_cold"] / peak,
                           "note": "hot = back-to-back launches, operands L2-resident as inside the step (the layer's "
                                   "working set is 26 MB); cold = L2 flushed before every launch"}
        out["roofline_kernels"] = rows
    step.close()   # the graph holds captured collectives: drop it before the process group goes away
    del step, model, opt
    gc.collect()
    torch.cuda.empty_cache()
    return out


# ----------------------------------------------------------------------------------------------------------
# packed-bit inference (second object of the line)
# ----------------------------------------------------------------------------------------------------------

def bench_packed(args, rank, world):
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
    packed = D.PackBitsTensor(host_bool.to(dev), bit_count=64)
    words0, pad = packed.t, packed.pad_len
    W = words0.shape[1]
    gates = [l._gate_ids() for l in layers]
    # two ping-pong activation buffers, allocated once (the API call allocates per layer)
    bufs = [torch.empty(EVAL_DIMS[1], W, dtype=torch.int64, device=dev) for _ in range(2)]

    # the plan PackBitsTensor.group_sum runs: all layers but the last one kernel each, then the last layer and the
    # group bit-sum in one kernel when its sizes are in that kernel's range
    fused_tail = os.environ.get("DL_FUSED_LAST_LAYER", "1") != "0" and ops.eval_groupbitsum_applicable(bufs[0], EVAL_DIMS[-1], EVAL_K)

    def run_resident():
        cur = words0
        last = len(layers) - 1
        for i, l in enumerate(layers):
            if i == last and fused_tail:
                return ops.eval_groupbitsum(cur, l.indices[0], l.indices[1], gates[i], pad, EVAL_K)
            cur = ops.eval_packed(cur, l.indices[0], l.indices[1], gates[i], out=bufs[i % 2])
        return ops.groupbitsum(cur, pad, EVAL_K)

    K, Wm = max(args.steps // 4, 5), 3
    for _ in range(Wm):
        run_resident()
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
    Ke = 3
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
        "value": EVAL_SAMPLES * K / t_dev, "ms_per_pass": t_dev / K * 1e3, "samples_per_gpu": local,
        "bytes_per_sample": eval_bytes_per_sample(EVAL_DIMS, EVAL_K, fused_tail),
        "bytes_per_sample_layer_by_layer": eval_bytes_per_sample(EVAL_DIMS, EVAL_K), "fused_last_layer": bool(fused_tail),
        "e2e": {"value": EVAL_SAMPLES * Ke / t_e2e, "unit": UNIT, "h2d_bytes_per_step": host_bool.numel(),
                "d2h_bytes_per_step": out_host.numel() * 4},
        "gpu_launches": launches, "clocks": sampler.summary(),
        "check": int(counts.sum().item()),
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
        }
        if fused_tail:
            kern["eval_groupbitsum"] = (8 * W * n + 4 * local * EVAL_K, lambda: L.dl_eval_groupbitsum(
                x.data_ptr(), l.indices[0].data_ptr(), l.indices[1].data_ptr(), gates[1].data_ptr(), out_counts.data_ptr(), n, n, W,
                pad, EVAL_K, 64, st))
        rows = {}
        for name, (nbytes, fn) in kern.items():
            for _ in range(2):
                fn()
            s, e = event_pair()
            s.record()
            for _ in range(10):
                fn()
            e.record()
            torch.cuda.synchronize()
            us = s.elapsed_time(e) * 1e3 / 10
            rows[name] = {"us": us, "bytes": nbytes, "achieved": nbytes / us / 1e3, "frac": nbytes / us / 1e3 / peak}
        res["roofline"] = {"kernel": "eval_kernel (8000 x 8000, %d int64 words per row)" % W, "bound": "hbm",
                           "achieved": rows["eval_packed"]["achieved"], "peak": peak, "unit": "GB/s",
                           "frac": rows["eval_packed"]["frac"], "peak_kind": peak_kind, "traffic": NCU_TRAFFIC["eval_packed"],
                           "algorithmic_bytes": rows["eval_packed"]["bytes"]}
        res["roofline_kernels"] = rows
    return res


# ----------------------------------------------------------------------------------------------------------
# CPU arms
# ----------------------------------------------------------------------------------------------------------

def cpu_train_steps(steps, warmup, budget_s=None):
    """The reference's CPU training step (implementation='python', device='cpu') as restated by the oracle, all host
    threads.  Returns (seconds, steps_done)."""
    from oracle import logic_oracle as O
    torch.manual_seed(0)
    net = O.OracleNet.build(TRAIN_DIMS, TRAIN_K, TRAIN_TAU)
    g = torch.Generator().manual_seed(1000)
    x = (torch.rand(TRAIN_BATCH, TRAIN_DIMS[0], generator=g) < P_ONE).float()
    y = torch.randint(0, TRAIN_K, (TRAIN_BATCH,), generator=g)
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


def cpu_packed_baseline(samples, threads):
    import numpy as np
    from oracle import logic_oracle as O
    torch.manual_seed(0)
    net = O.OracleNet.build(EVAL_DIMS, EVAL_K, EVAL_TAU)
    x = (torch.rand(samples, EVAL_DIMS[0], generator=torch.Generator().manual_seed(5)) < P_ONE).numpy()
    gates = net.gate_ids()
    O.c_packed_net_counts(x[:4096], net.idx_a, net.idx_b, gates, EVAL_K, threads)
    t0 = time.perf_counter()
    out = O.c_packed_net_counts(x, net.idx_a, net.idx_b, gates, EVAL_K, threads)
    dt = time.perf_counter() - t0
    return samples / dt, int(np.asarray(out).sum())


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = torch.get_num_threads()
    t, done = cpu_train_steps(args.steps, max(args.warmup, 1))
    value = TRAIN_BATCH * done / t
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": done,
        "warmup": max(args.warmup, 1), "ms_per_step": t / done * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "train step, 784 -> 5 x 16000 -> GroupSum(10, tau=30), batch 128, CPU"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": "%d full training steps at batch 128 with torch on %d host threads" % (done, cores)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------------------

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--loss", default="fused", choices=["fused", "torch"],
                    help="fused: difflogic_b200.losses.CrossEntropyLoss (one kernel each way); torch: torch.nn.CrossEntropyLoss")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="N > 1: peer = gradient exchange + Adam in one kernel over peer memory; nccl = NCCL all-reduce")
    ap.add_argument("--skip-packed", action="store_true")
    ap.add_argument("--optimizer", default="flat", choices=["flat", "torch"],
                    help="flat: difflogic_b200.optim.FlatAdam (one kernel); torch: torch.optim.Adam(capturable, fused)")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--no-flush", action="store_true", help="diagnostic only: do not flush L2 between the timed steps")
    ap.add_argument("--buckets", type=int, default=2, help="all-reduce pieces of the flat gradient buffer (N > 1)")
    ap.add_argument("--skip-kernel-timing", action="store_true", help="leave out the per-kernel roofline timing")
    args = ap.parse_args()
    # a run that is stuck (e.g. in a collective) ends itself with a traceback instead of holding the GPUs
    faulthandler.dump_traceback_later(1200, exit=True)

    if args.impl == "reference":
        reference_arm(args)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"   # keep NCCL's version banner out of stdout: one JSON line only
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    assert world == args.gpus or world == 1, "launch with torchrun --nproc-per-node %d" % args.gpus

    import __graft_entry__
    if rank == 0:
        __graft_entry__.build()
    barrier(world)

    train = bench_train(args, rank, world)
    packed = None if args.skip_packed else bench_packed(args, rank, world)

    if rank == 0:
        line = {
            "metric": METRIC, "value": train["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": train["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "train step: Flatten -> LogicLayer(784,16000) -> 4 x LogicLayer(16000,16000) -> "
                                   "GroupSum(10, tau=30), CrossEntropy, Adam lr=0.01",
                       "batch_per_gpu": TRAIN_BATCH, "global_batch": TRAIN_BATCH * world,
                       "parallelism": "batch-sharded replicas x%d, weight-gradient exchange: %s" % (
                           world, "none" if world == 1 else ("reduce-scatter + Adam + all-gather in one kernel over peer memory"
                                                             if args.exchange == "peer" and args.optimizer == "flat" else "NCCL all-reduce")),
                       "execution": "whole step replayed as one CUDA graph",
                       "loss": "CrossEntropy (%s)" % ("difflogic_b200.losses.CrossEntropyLoss" if args.loss == "fused"
                                                      else "torch.nn.CrossEntropyLoss"),
                       "optimizer": "Adam lr=0.01 (%s)" % ("difflogic_b200.optim.FlatAdam" if args.optimizer == "flat"
                                                           else "torch.optim.Adam capturable fused"),
                       "l2": "flushed between timed steps (256 MiB memset, untimed)"},
            "e2e": train["e2e"], "gpu_launches": train["gpu_launches"], "launches_per_step": train["launches_per_step"],
            "exchange_kernel_last_step": train["exchange_kernel_last_step"],
            "clocks": train["clocks"], "loss": train["loss"],
            "step_algorithmic_bytes": train["step_algorithmic_bytes"], "step_hbm_frac": train["step_hbm_frac"],
            "roofline": train.get("roofline"), "roofline_kernels": train.get("roofline_kernels"),
        }
        if packed is not None:
            line["packed_eval"] = packed
        if not args.skip_cpu and world == 1:
            cores = torch.get_num_threads()
            t, done = cpu_train_steps(5, 1, budget_s=20.0)
            line["cpu_baseline"] = {"value": TRAIN_BATCH * done / t, "unit": UNIT, "cores": cores, "kind": "port",
                                    "sample": "%d training steps of the same net at batch 128 (oracle restatement of the "
                                              "reference's implementation='python' CPU path)" % done}
            if packed is not None:
                v, _ = cpu_packed_baseline(1 << 17, cores)
                v1, _ = cpu_packed_baseline(1 << 14, 1)
                packed["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "single_core_value": v1,
                                          "sample": "2^17 samples through the C oracle (table-driven restatement of "
                                                    "CompiledLogicNet's generated C, num_bits=64)"}
        print(json.dumps(line))
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
