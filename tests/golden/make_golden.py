"""Generates the golden fixtures in this folder from the reference implementation.

Run where the reference checkout is available (it is NOT needed to run the tests):

    python tests/golden/make_golden.py /path/to/reference

The reference's pure-python CPU path (implementation='python', device='cpu') and its
CompiledLogicNet C build (gcc) are imported unmodified; its native CUDA module is replaced by an
empty stand-in because it is only needed for implementation='cuda'.  The outputs are stored as
small .npz files; the seeds used here are re-used by the tests to regenerate the same models.
"""
import io
import contextlib
import sys
import types

import numpy as np
import torch


def load_reference(path):
    sys.modules["difflogic_cuda"] = types.ModuleType("difflogic_cuda")
    sys.path.insert(0, path)
    import difflogic  # noqa
    from difflogic import functional
    return difflogic, functional


def quiet(fn, *a, **kw):
    with contextlib.redirect_stdout(io.StringIO()):
        return fn(*a, **kw)


def build(difflogic, dims, k, tau, grad_factor=1.0, connections="random"):
    layers = [torch.nn.Flatten()]
    for n_in, n_out in zip(dims[:-1], dims[1:]):
        layers.append(difflogic.LogicLayer(n_in, n_out, device="cpu", implementation="python",
                                           grad_factor=grad_factor, connections=connections))
    layers.append(difflogic.GroupSum(k, tau, device="cpu"))
    return torch.nn.Sequential(*layers)


def logic_layers(model):
    return [m for m in model if hasattr(m, "indices")]


def train_and_eval(difflogic, model, x, y, lr=0.01, compiled_bits=(64,), opt_level=0):
    out = {}
    model.train()
    opt = torch.optim.Adam(model.parameters(), lr=lr)
    w0 = [l.weights.detach().clone() for l in logic_layers(model)]
    logits = quiet(model, x)
    loss = torch.nn.functional.cross_entropy(logits, y)
    opt.zero_grad()
    loss.backward()
    grads = [l.weights.grad.detach().clone() for l in logic_layers(model)]
    # eval + compiled net on the PRE-step weights (restored below)
    opt.step()
    w1 = [l.weights.detach().clone() for l in logic_layers(model)]
    out.update(train_logits=logits.detach().numpy(), loss=np.float32(loss.item()))
    model.eval()
    with torch.no_grad():
        out["eval_logits_after_step"] = quiet(model, x).numpy()
        for l, w in zip(logic_layers(model), w0):
            l.weights.copy_(w)
        out["eval_logits"] = quiet(model, x).numpy()
    for bits in compiled_bits:
        net = difflogic.CompiledLogicNet(model, num_bits=bits, cpu_compiler="gcc")
        quiet(net.compile, opt_level=opt_level)
        out["compiled_counts_%d" % bits] = net.forward(x.bool().numpy()).numpy().astype(np.int32)
    return out, w0, w1, grads


def main(ref_path, out_dir):
    difflogic, functional = load_reference(ref_path)

    # ---- 1. the 16 relaxed gates and their weighted mix --------------------------------------
    torch.manual_seed(11)
    a = torch.rand(5, 13)
    b = torch.rand(5, 13)
    w = torch.softmax(torch.randn(5, 13, 16), -1)
    gates = torch.stack([functional.bin_op(a, b, i) for i in range(16)])
    np.savez(out_dir + "/gates.npz", a=a.numpy(), b=b.numpy(), w=w.numpy(), gates=gates.numpy(),
             mix=functional.bin_op_s(a, b, w).numpy())

    # ---- 2. a small ragged net, everything stored ---------------------------------------------
    for name, dims, k, tau, B, gf, seed in (("small_net", [20, 32, 30], 3, 2.0, 37, 1.0, 1),
                                            ("small_net_gf2", [12, 40, 40, 36], 2, 5.0, 70, 2.0, 2)):
        torch.manual_seed(seed)
        model = build(difflogic, dims, k, tau, gf)
        x = (torch.rand(B, dims[0]) < 0.4).float()
        y = torch.randint(0, k, (B,))
        # grad wrt the input as well (needs backward_x of layer 1)
        xr = x.clone().requires_grad_(True)
        model.train()
        lg = quiet(model, xr)
        torch.nn.functional.cross_entropy(lg, y).backward()
        grad_x = xr.grad.detach().clone()
        for l in logic_layers(model):
            l.weights.grad = None
        out, w0, w1, grads = train_and_eval(difflogic, model, x, y, compiled_bits=(8, 16, 32, 64))
        d = dict(out, x=x.numpy(), y=y.numpy(), grad_x=grad_x.numpy(), dims=np.array(dims), k=k, tau=tau,
                 grad_factor=gf, seed=seed)
        for i, l in enumerate(logic_layers(model)):
            d["w0_%d" % i] = w0[i].numpy()
            d["w1_%d" % i] = w1[i].numpy()
            d["grad_%d" % i] = grads[i].numpy()
            d["a_%d" % i] = l.indices[0].numpy()
            d["b_%d" % i] = l.indices[1].numpy()
        np.savez(out_dir + "/%s.npz" % name, **d)

    # ---- 3. config 1 (4 layers of 8000), regenerated from seed 0 by the tests ----------------
    torch.manual_seed(0)
    dims = [784, 8000, 8000, 8000, 8000]
    model = build(difflogic, dims, 10, 10.0)
    x = (torch.rand(100, 784) < 0.19).float()
    y = torch.randint(0, 10, (100,))
    out, w0, w1, grads = train_and_eval(difflogic, model, x, y, compiled_bits=(64,), opt_level=0)
    g = torch.Generator().manual_seed(123)
    d = dict(out, y=y.numpy(), x_rowsum=x.sum(1).numpy())
    for i, l in enumerate(logic_layers(model)):
        pos = torch.randint(0, grads[i].numel(), (256,), generator=g)
        d["pos_%d" % i] = pos.numpy()
        d["grad_sample_%d" % i] = grads[i].reshape(-1)[pos].numpy()
        d["grad_absmax_%d" % i] = np.float32(grads[i].abs().max().item())
        d["grad_sum_%d" % i] = np.float64(grads[i].double().sum().item())
        d["w1_sample_%d" % i] = w1[i].reshape(-1)[pos].numpy()
        d["w0_sample_%d" % i] = w0[i].reshape(-1)[pos].numpy()
        ar = torch.arange(l.indices[0].numel())
        d["idx_check_%d" % i] = np.array([(l.indices[0] * ar).sum().item(), (l.indices[1] * ar).sum().item()])
    np.savez(out_dir + "/config1.npz", **d)

    # ---- 4. 'unique' connections ---------------------------------------------------------------
    d = {}
    for j, (n_in, n_out) in enumerate(((10, 5), (10, 9), (10, 30), (7, 20), (16, 16), (9, 36))):
        torch.manual_seed(100 + j)
        a_, b_ = functional.get_unique_connections(n_in, n_out, "cpu")
        d["a_%d" % j] = a_.numpy()
        d["b_%d" % j] = b_.numpy()
        d["dims_%d" % j] = np.array([n_in, n_out])
    np.savez(out_dir + "/unique_connections.npz", **d)
    print("fixtures written to", out_dir)


if __name__ == "__main__":
    import os
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/reference")
    main(sys.argv[1], os.path.dirname(os.path.abspath(__file__)))
