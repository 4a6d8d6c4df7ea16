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

    # -- batch-sharded training: exchange and step in one kernel over peer memory -------------------------------

    def enable_exchange(self, group=None):
        """Switches to the peer-memory exchange (dl_adam_exchange_step_f32): the flat parameter and gradient buffers
        move into memory that the other ranks of `group` (one process per GPU on this machine) map through CUDA IPC;
        `step()` then averages the gradients over the ranks, applies Adam to this rank's slice and distributes the new
        parameters in a single kernel.  No NCCL call is made per step.  Collective: every rank of the group calls it."""
        import ctypes
        import torch.distributed as dist
        lib = N.lib()
        world = dist.get_world_size(group)
        rank = dist.get_rank(group)
        dev = self.flat_param.device
        n = self.flat_param.numel()
        assert n % 4 == 0

        def alloc(nbytes):
            ptr = ctypes.c_void_p()
            with torch.cuda.device(dev):
                N.check(lib.dl_comm_alloc(nbytes, ctypes.byref(ptr)))
            return ptr.value

        def as_tensor(ptr, count, typestr, dtype):
            holder = type("_Raw", (), {})()
            holder.__cuda_array_interface__ = {"shape": (count,), "typestr": typestr, "data": (ptr, False), "version": 2}
            t = torch.as_tensor(holder, device=dev)
            assert t.dtype == dtype and t.data_ptr() == ptr
            return t

        ptrs = {"param": alloc(n * 4), "grad": alloc(n * 4), "flags": alloc(256)}
        new_param = as_tensor(ptrs["param"], n, "<f4", torch.float32)
        new_grad = as_tensor(ptrs["grad"], n, "<f4", torch.float32)
        with torch.no_grad():
            new_param.copy_(self.flat_param)
            dist.broadcast(new_param, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
            for p in self._params:
                off, cnt = self._slices[p]
                p.data = new_param[off:off + cnt].view_as(p)
                p._dl_grad_out = new_grad[off:off + cnt].view_as(p)
        self.flat_param, self.flat_grad = new_param, new_grad

        handles = {}
        for name, ptr in ptrs.items():
            buf = (ctypes.c_ubyte * 64)()
            N.check(lib.dl_comm_export(ptr, buf))
            handles[name] = bytes(buf)
        gathered = [None] * world
        dist.all_gather_object(gathered, handles, group=group)
        self._peer_ptrs = {}
        for name in ptrs:
            arr = (ctypes.c_void_p * world)()
            for r in range(world):
                if r == rank:
                    arr[r] = ptrs[name]
                else:
                    out = ctypes.c_void_p()
                    with torch.cuda.device(dev):
                        N.check(lib.dl_comm_import(gathered[r][name], ctypes.byref(out)))
                    arr[r] = out.value
            self._peer_ptrs[name] = arr
        per = -(-(n // 4) // world) * 4
        self.exp_avg = torch.zeros(per, dtype=torch.float32, device=dev)       # moments of this rank's slice only
        self.exp_avg_sq = torch.zeros(per, dtype=torch.float32, device=dev)
        self.state_t = torch.zeros(16, dtype=torch.int32, device=dev)
        self._exchange = (rank, world)
        self.exchange_enabled = True
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)
        return self

    def exchange_error(self):
        """True when a wait for a peer ever ran out of its poll limit (synchronises)."""
        return bool(int(self.state_t[2].item())) if getattr(self, "exchange_enabled", False) else False

    def exchange_timing(self):
        """Nanoseconds inside the latest exchange kernel on this rank (synchronises): waiting for all ranks' gradients,
        reduce + Adam on this rank's slice, waiting for all ranks' slices, fetching the other slices."""
        if not getattr(self, "exchange_enabled", False):
            return None
        t = self.state_t[4:16].cpu().view(torch.int64).tolist()
        return {"wait_gradients_ns": t[1] - t[0], "slice_ns": t[2] - t[1], "wait_slices_ns": t[3] - t[2], "gather_ns": t[5] - t[3],
                "total_ns": t[5] - t[0], "first_block_slice_ns": t[4] - t[1]}

    # -- Adam inside backward_w ---------------------------------------------------------------------------------------

    def enable_step_in_backward(self, on=True):
        """With `on`, every LogicLayer whose weights this optimizer holds applies the Adam update in the epilogue of its
        backward_w kernel (a neuron's 16 gradients go from registers straight into the update); `loss.backward()`
        then UPDATES the weights and stores no gradient, and the caller must not call `step()` for that pass
        (`TrainStep` handles this).  Every parameter counts its own steps on the device (`layer_state`);
        `sync_step_counts()` carries the count over when the way of stepping changes.  Single GPU only."""
        if on and getattr(self, "exchange_enabled", False):
            raise RuntimeError("FlatAdam: the step inside backward_w and the peer-memory exchange exclude each other")
        if on and getattr(self, "layer_state", None) is None:
            self.layer_state = torch.zeros((len(self._params), 2), dtype=torch.int32, device=self.flat_param.device)
            self._layer_index = {p: i for i, p in enumerate(self._params)}
            self.sync_step_counts(to_layers=True)
        for p in self._params:
            p._dl_adam = self if on else None
        return self

    @torch.no_grad()
    def sync_step_counts(self, to_layers):
        """to_layers: every parameter's own count := the optimizer's count (before stepping inside backward_w);
        else the optimizer's count := the first parameter's (before stepping with `step()` again)."""
        if getattr(self, "layer_state", None) is None:
            return
        if to_layers:
            self.layer_state[:, 0] = self.state_t[0]
        else:
            self.state_t[0] = self.layer_state[0, 0]

    def backward_args(self, p):
        """What ops.logic_backward_w_adam needs for parameter p: its moment slices, its step count and the hyper-parameters."""
        off, cnt = self._slices[p]
        g = self.param_groups[0]
        beta1, beta2 = g['betas']
        return dict(exp_avg=self.exp_avg[off:off + cnt], exp_avg_sq=self.exp_avg_sq[off:off + cnt],
                    state=self.layer_state[self._layer_index[p]], lr=g['lr'], beta1=beta1, beta2=beta2, eps=g['eps'],
                    grad_scale=self.grad_scale)

    def prefetch_state(self):
        """Launches (on the current stream) a kernel that pulls the moments towards L2.  They are touched once per step,
        so a step that begins with a cold L2 otherwise reads them from HBM at the very end, after the last gradient."""
        with torch.cuda.device(self.flat_param.device):
            st = N.stream_of(self.flat_param)
            for t in (self.exp_avg, self.exp_avg_sq):
                N.check(N.lib().dl_prefetch_l2(t.data_ptr(), t.numel() * 4, st))

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
        if getattr(self, "exchange_enabled", False):
            rank, world = self._exchange
            with torch.cuda.device(self.flat_param.device):
                N.check(N.lib().dl_adam_exchange_step_f32(self._peer_ptrs["param"], self._peer_ptrs["grad"],
                                                          self._peer_ptrs["flags"], rank, world, self.exp_avg.data_ptr(),
                                                          self.exp_avg_sq.data_ptr(), self.flat_param.numel(), float(g['lr']),
                                                          float(beta1), float(beta2), float(g['eps']),
                                                          self.state_t.data_ptr(), N.stream_of(self.flat_param)))
            return loss
        with torch.cuda.device(self.flat_param.device):
            N.check(N.lib().dl_adam_step_f32(self.flat_param.data_ptr(), self.flat_grad.data_ptr(), self.exp_avg.data_ptr(),
                                             self.exp_avg_sq.data_ptr(), self.flat_param.numel(), float(g['lr']), float(beta1),
                                             float(beta2), float(g['eps']), float(self.grad_scale), self.state_t.data_ptr(),
                                             N.stream_of(self.flat_param)))
        return loss
