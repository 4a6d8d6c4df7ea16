"""Host-side logic of the multi-GPU paths, exercised with world_size-2 gloo process groups on the CPU:
batch-sharded training equals one step on the concatenated batch, and batch shards of the packed-bit
inference concatenate to the unsharded result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import logic_oracle as O
from tests.helpers import build_model, logic_layers


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _train_worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from difflogic_b200.training import TrainStep, shard_range
        torch.manual_seed(0)
        dims = [24, 48, 40]
        net = O.OracleNet.build(dims, 4, 3.0)
        model = build_model(dims, 4, 3.0, net.weights, net.idx_a, net.idx_b, device="cpu")
        model.train()
        g = torch.Generator().manual_seed(7)
        x = (torch.rand(32, 24, generator=g) < 0.4).float()
        y = torch.randint(0, 4, (32,), generator=g)
        lo, hi = shard_range(32, rank, world)
        step = TrainStep(model, torch.optim.Adam(model.parameters(), lr=0.01), process_group=dist.group.WORLD)
        loss = step(x[lo:hi], y[lo:hi])
        torch.save({"loss": loss, "weights": [l.weights.detach().clone() for l in logic_layers(model)]},
                   os.path.join(out_dir, "rank%d.pt" % rank))
    finally:
        dist.destroy_process_group()


def test_sharded_training_step_equals_full_batch_step(tmp_path):
    world = 2
    mp.spawn(_train_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    r0 = torch.load(os.path.join(tmp_path, "rank0.pt"))
    r1 = torch.load(os.path.join(tmp_path, "rank1.pt"))
    # replicas stay identical
    for w0, w1 in zip(r0["weights"], r1["weights"]):
        assert torch.equal(w0, w1)
    # and equal to a single step on the whole batch
    torch.manual_seed(0)
    dims = [24, 48, 40]
    net = O.OracleNet.build(dims, 4, 3.0)
    g = torch.Generator().manual_seed(7)
    x = (torch.rand(32, 24, generator=g) < 0.4).float()
    y = torch.randint(0, 4, (32,), generator=g)
    loss, _, _ = net.train_step(x, y)
    assert abs(0.5 * (float(r0["loss"]) + float(r1["loss"])) - float(loss)) < 1e-6
    for w, ref in zip(r0["weights"], net.weights):
        assert torch.allclose(w, ref.detach(), rtol=1e-5, atol=1e-6)


def test_shard_range_covers_the_batch_in_whole_words():
    from difflogic_b200.training import shard_range
    for n, world in ((1 << 20, 8), (1000, 4), (64, 8), (130, 2), (5, 3)):
        pieces = [shard_range(n, r, world, multiple=64) for r in range(world)]
        assert pieces[0][0] == 0 and pieces[-1][1] == n
        for (a0, a1), (b0, b1) in zip(pieces, pieces[1:]):
            assert a1 == b0 and a0 <= a1
        for lo, hi in pieces:
            assert hi == lo or (lo % 64 == 0 and (hi % 64 == 0 or hi == n))


def test_packed_inference_shards_concatenate_bit_exact():
    from difflogic_b200.training import shard_range
    torch.manual_seed(3)
    net = O.OracleNet.build([50, 128, 120], 10, 1.0)
    x = (torch.rand(1000, 50) < 0.3).numpy()
    full = O.packed_net_counts(x, net.idx_a, net.idx_b, net.gate_ids(), 10, 64)
    parts = []
    for r in range(4):
        lo, hi = shard_range(1000, r, 4, multiple=64)
        if hi > lo:
            parts.append(O.c_packed_net_counts(x[lo:hi], net.idx_a, net.idx_b, net.gate_ids(), 10))
    assert np.array_equal(np.concatenate(parts), full)
