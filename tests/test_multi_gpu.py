"""Batch-sharded training on more than one GPU: the peer-memory exchange (two kernels per layer, launched beside the
backward pass) against the NCCL all-reduce path and against the oracle's step on the whole batch.
Runs child processes, one per GPU; skipped where fewer than two GPUs are visible.  The single-rank case of the
exchange kernels (no peers) runs on one GPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import logic_oracle as O
from tests.helpers import build_model, logic_layers

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _make(dims, k, tau, seed):
    torch.manual_seed(seed)
    net = O.OracleNet.build(dims, k, tau)
    return net, build_model(dims, k, tau, net.weights, net.idx_a, net.idx_b)


def test_exchange_kernel_single_rank_equals_flat_adam(tmp_path):
    from difflogic_b200.optim import FlatAdam
    dist.init_process_group("gloo", init_method="file://%s" % (tmp_path / "store"), rank=0, world_size=1)
    try:
        dims = [30, 64, 52]
        _, m1 = _make(dims, 4, 2.0, 5)
        _, m2 = _make(dims, 4, 2.0, 5)
        o1 = FlatAdam(m1.parameters(), lr=0.01)
        o2 = FlatAdam(m2.parameters(), lr=0.01).enable_exchange(dist.group.WORLD)
        x = (torch.rand(40, 30, generator=torch.Generator().manual_seed(1)) < 0.5).float().cuda()
        y = torch.randint(0, 4, (40,), generator=torch.Generator().manual_seed(2)).cuda()
        for _ in range(4):
            for m, o in ((m1, o1), (m2, o2)):
                m.train()
                loss = torch.nn.functional.cross_entropy(m(x), y)
                o.zero_grad()
                loss.backward()
                o.step()
        for l1, l2 in zip(logic_layers(m1), logic_layers(m2)):
            assert torch.equal(l1.weights, l2.weights)
        assert not o2.exchange_error() and o2.state_t[:, 0].tolist() == [4] * len(logic_layers(m2))
        o2.close()
        assert all(l.weights.data_ptr() != 0 for l in logic_layers(m2))
    finally:
        dist.destroy_process_group()


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from difflogic_b200.optim import FlatAdam
        from difflogic_b200.training import TrainStep, shard_range
        dims = [24, 160, 160, 80]
        g = torch.Generator().manual_seed(3)
        xs = [(torch.rand(64, 24, generator=g) < 0.4).float() for _ in range(3)]
        ys = [torch.randint(0, 4, (64,), generator=g) for _ in range(3)]
        lo, hi = shard_range(64, rank, world)
        results = {}
        # peer, peer_graph: the default forms (these buckets are small: packets, pushed by the exchange kernel);
        # peer_push: packets pushed by backward_w itself; peer_flags: the flag exchange, in one pass where the byte
        # limit allows; peer_two_pass_announce: the flag exchange in two passes, announced by backward_w
        for mode in ("nccl", "peer", "peer_graph", "peer_push", "peer_flags", "peer_two_pass_announce"):
            _, model = _make(dims, 4, 3.0, 11)
            model.train()
            opt = FlatAdam(model.parameters(), lr=0.01)
            if mode == "peer_two_pass_announce":   # every bucket in two passes, gradients announced by backward_w itself
                opt.enable_exchange(dist.group.WORLD, announce_in_backward=True, one_pass_bytes=0, packet_bytes=0)
            elif mode == "peer_flags":
                opt.enable_exchange(dist.group.WORLD, packet_bytes=0)
            elif mode == "peer_push":
                opt.enable_exchange(dist.group.WORLD, push_in_backward=True)
            elif mode != "nccl":
                opt.enable_exchange(dist.group.WORLD)
            step = TrainStep(model, opt, process_group=dist.group.WORLD, buckets=1)
            if mode == "peer_graph":
                step.capture(xs[0][lo:hi].cuda(), ys[0][lo:hi].cuda(), warmup=0)
            losses, first = [], None
            for x, y in zip(xs, ys):
                if mode == "peer":
                    opt.rank_barrier()     # the ranks meet on the device in front of the step; an error shows in "err"
                losses.append(float(step(x[lo:hi].cuda(), y[lo:hi].cuda()).item()))
                if first is None:
                    first = {"w": [l.weights.detach().cpu().clone() for l in logic_layers(model)]}
                    if mode != "nccl":
                        # first moments after one step from zero are (1 - beta1) * averaged gradient; every rank holds its slices
                        m = opt.full_exp_avg()
                        first["grad"] = [(m[off:off + cnt] / 0.1).view_as(p).cpu() for p in opt._params
                                         for off, cnt in [opt._slices[p]]]
            torch.cuda.synchronize()
            results[mode] = {"loss": losses, "w": [l.weights.detach().cpu().clone() for l in logic_layers(model)],
                             "err": opt.exchange_error(), "first": first}
            step.close()
            dist.barrier()
        torch.save(results, os.path.join(out_dir, "rank%d.pt" % rank))
    finally:
        torch.cuda.synchronize()
        dist.barrier()
        os._exit(0)  # skip the NCCL teardown (it can block while graphs with captured kernels are alive)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_memory_exchange_matches_nccl_all_reduce(tmp_path):
    world = 2
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, str(tmp_path))) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    for p in procs:
        if p.is_alive():
            p.kill()
            pytest.fail("a rank did not finish in time")
        assert p.exitcode == 0
    res = [torch.load(os.path.join(tmp_path, "rank%d.pt" % r)) for r in range(world)]
    for mode in ("peer", "peer_graph", "peer_push", "peer_flags", "peer_two_pass_announce"):
        assert not res[0][mode]["err"] and not res[1][mode]["err"]
        for w0, w1 in zip(res[0][mode]["w"], res[1][mode]["w"]):
            assert torch.equal(w0, w1)                       # replicas stay identical
        for w, ref in zip(res[0][mode]["w"], res[0]["nccl"]["w"]):
            assert torch.allclose(w, ref, rtol=1e-5, atol=1e-6)   # same update as all-reduce + Adam
    assert torch.allclose(torch.tensor(res[0]["peer"]["loss"]), torch.tensor(res[0]["nccl"]["loss"]), rtol=1e-5)

    # against the oracle: the same three steps on the WHOLE batch (experiments/main.py:174-181) with torch's Adam
    from tests.helpers import assert_grad_close
    dims = [24, 160, 160, 80]
    torch.manual_seed(11)
    net = O.OracleNet.build(dims, 4, 3.0)
    start = [w.detach().clone() for w in net.weights]
    g = torch.Generator().manual_seed(3)
    xs = [(torch.rand(64, 24, generator=g) < 0.4).float() for _ in range(3)]
    ys = [torch.randint(0, 4, (64,), generator=g) for _ in range(3)]
    adam = torch.optim.Adam(net.weights, lr=0.01)
    ref_losses, ref_first_grads = [], None
    for x, y in zip(xs, ys):
        loss = torch.nn.functional.cross_entropy(net.forward(x, True), y)
        adam.zero_grad()
        loss.backward()
        if ref_first_grads is None:
            ref_first_grads = [w.grad.detach().clone() for w in net.weights]
        adam.step()
        ref_losses.append(float(loss))
    for mode in ("peer", "peer_graph", "peer_push", "peer_flags", "peer_two_pass_announce"):
        mean_losses = [0.5 * (a + b) for a, b in zip(res[0][mode]["loss"], res[1][mode]["loss"])]   # equal shards
        assert torch.allclose(torch.tensor(mean_losses), torch.tensor(ref_losses), rtol=1e-4), (mode, mean_losses, ref_losses)
        for got, ref in zip(res[0][mode]["first"]["grad"], ref_first_grads):
            assert_grad_close(got, ref, "%s: averaged gradient of the first step" % mode)
        for w, w0, gr in zip(res[0][mode]["first"]["w"], start, ref_first_grads):
            want = w0 - 0.01 * gr / (gr.abs() + 1e-8)       # first Adam step from zero moments
            moved = gr.abs() > 1e-3 * gr.abs().max()        # where the sign of the gradient is beyond doubt
            assert (w - want)[moved].abs().max().item() <= 2e-3 * 0.01
