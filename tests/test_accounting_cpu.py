"""Byte accounting and host-side choices that need no GPU."""
import importlib.util
import os

import torch

import difflogic_b200 as D
from difflogic_b200.training import TrainStep

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_algorithmic_bytes_of_the_baseline_configurations():
    # per-GPU figures of the baseline's table: config 2, 4 and 5 training steps, config 3 and 5 packed inference
    bench = _bench()
    total, per_kernel = bench.train_bytes_per_step(bench.TRAIN_DIMS, bench.TRAIN_BATCH, bench.TRAIN_K)
    assert total == 343_853_088
    assert per_kernel["forward"] == 17_664_000 and per_kernel["backward_x"] == 26_240_008
    c4, c5 = bench.CONFIGS["c4"], bench.CONFIGS["c5"]
    assert bench.train_bytes_per_step(c4["dims"], c4["batch"], c4["k"])[0] == 3_810_766_872
    assert bench.train_bytes_per_step(c5["dims"], c5["batch"], c5["k"])[0] == 22_021_697_624
    assert bench.eval_bytes_per_sample(bench.EVAL_DIMS, bench.EVAL_K, False) == 8138
    assert bench.eval_bytes_per_sample(bench.EVAL_DIMS, bench.EVAL_K, True) == 6138
    assert bench.eval_bytes_per_sample(c5["dims"], c5["k"], False) == 192_040


def test_both_bench_arms_name_the_same_configuration():
    bench = _bench()
    assert bench.train_config(4) == bench.train_config(4) and bench.train_config(1)["global_batch"] == 128
    assert bench.train_config(8)["global_batch"] == 1024


def test_train_step_fuses_the_head_only_for_a_default_cross_entropy():
    model = torch.nn.Sequential(torch.nn.Flatten(), D.LogicLayer(8, 16, device='cpu', implementation='python'),
                                D.GroupSum(2))
    fus = TrainStep._head_is_fusable
    assert fus(model, torch.nn.CrossEntropyLoss())
    assert fus(model, D.losses.CrossEntropyLoss()) if hasattr(D, "losses") else True
    assert not fus(model, torch.nn.CrossEntropyLoss(label_smoothing=0.1))
    assert not fus(model, torch.nn.CrossEntropyLoss(reduction="sum"))
    assert not fus(model, torch.nn.MSELoss())
    assert not fus(model[:-1], torch.nn.CrossEntropyLoss())                 # no GroupSum at the end
    # on the CPU nothing is fused and the step is the plain one
    opt = torch.optim.Adam(model.parameters(), lr=0.01)
    step = TrainStep(model, opt, torch.nn.CrossEntropyLoss())
    assert step._head is None and not step._in_backward
    x = (torch.rand(6, 8) < 0.5).float()
    y = torch.randint(0, 2, (6,))
    before = model[1].weights.detach().clone()
    loss = step(x, y)
    assert loss.ndim == 0 and not torch.equal(before, model[1].weights.detach())
