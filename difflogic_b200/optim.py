"""Flat-buffer Adam for logic gate networks.

`FlatAdam` moves the parameters it is given into one flat fp32 buffer (each parameter becomes a view
of it), keeps the gradients, first and second moments in flat buffers of the same layout and performs
the Adam update of the whole network with one kernel (dl_adam_step_f32).  The update rule is that of
torch.optim.Adam(lr, betas, eps) without weight decay or amsgrad, which is what the reference's
training loop uses (experiments/main.py:169).

LogicLayer's backward writes each layer's weight gradient straight into its slice of the flat
gradient buffer (`grad_view(param)`), so in data-parallel training the buffer can be all-reduced as it
is and no gradient is copied.  The step counter lives on the device: a step can be captured in a CUDA
graph and replayed.
"""
import torch

from . import _native as N


class FlatAdam(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8):
        defaults = dict(lr=lr, betas=betas, eps=eps)
        super().__init__(params, defaults)
        plist = [p for g in self.param_groups for p in g['params']]
        if len(self.param_groups) != 1:
            raise ValueError("FlatAdam supports a single parameter group")
        if not plist:
            raise ValueError("FlatAdam got an empty parameter list")
        dev = plist[0].device
        for p in plist:
            if not (p.is_cuda and p.dtype == torch.float32 and p.device == dev):
                raise ValueError("FlatAdam needs float32 CUDA parameters on one device")
        self._params = plist
        sizes = [(p.numel() + 3) // 4 * 4 for p in plist]  # keep every slice 16-byte aligned
        total = sum(sizes)
        self.flat_param = torch.zeros(total, dtype=torch.float32, device=dev)
        self.flat_grad = torch.zeros(total, dtype=torch.float32, device=dev)
        self.exp_avg = torch.zeros(total, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(total, dtype=torch.float32, device=dev)
        self.state_t = torch.zeros(2, dtype=torch.int32, device=dev)  # {steps done, ticket}
        self._slices = {}
        off = 0
        with torch.no_grad():
            for p, sz in zip(plist, sizes):
                view = self.flat_param[off:off + p.numel()].view_as(p)
                view.copy_(p)
                p.data = view
                self._slices[p] = (off, p.numel())
                p._dl_grad_out = self.flat_grad[off:off + p.numel()].view_as(p)  # LogicLayer's backward_w writes here
                off += sz
        self.grad_scale = 1.0

    def grad_view(self, p):
        off, n = self._slices[p]
        return self.flat_grad[off:off + n].view_as(p)

    def zero_grad(self, set_to_none=True):
        # gradients are fully overwritten by backward_w every step; dropping the references is enough
        for p in self._params:
            p.grad = None

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        # a gradient that did not land in the flat buffer (a parameter that is not a LogicLayer weight) is copied in
        for p in self._params:
            if p.grad is not None and p.grad.data_ptr() != self.grad_view(p).data_ptr():
                self.grad_view(p).copy_(p.grad)
        g = self.param_groups[0]
        beta1, beta2 = g['betas']
        with torch.cuda.device(self.flat_param.device):
            N.check(N.lib().dl_adam_step_f32(self.flat_param.data_ptr(), self.flat_grad.data_ptr(), self.exp_avg.data_ptr(),
                                             self.exp_avg_sq.data_ptr(), self.flat_param.numel(), float(g['lr']), float(beta1),
                                             float(beta2), float(g['eps']), float(self.grad_scale), self.state_t.data_ptr(),
                                             N.stream_of(self.flat_param)))
        return loss
