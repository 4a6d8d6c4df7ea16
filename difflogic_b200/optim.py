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

    # -- batch-sharded training: exchange and step over peer memory, bucket by bucket -------------------------------

    def enable_exchange(self, group=None, buckets=None, poll_limit=0):
        """Switches to the peer-memory exchange (dl_exchange_reduce_adam_f32 / dl_exchange_gather_f32): the flat
        parameter and gradient buffers move into memory that the other ranks of `group` (one process per GPU on this
        machine) map through CUDA IPC.  The buffers are cut into buckets -- one per parameter, or `buckets` groups of
        consecutive parameters.  As soon as the backward_w kernels of a bucket's layers have been launched, the
        bucket's two exchange kernels are launched on a stream of their own: the gradients are averaged over the
        ranks, Adam is applied to this rank's slice, the new parameters are fetched from the other ranks, all beside
        the rest of the backward pass.  `step()` launches whatever is still missing and makes the current stream wait
        for the exchange.  No NCCL call is made per step.  Collective: every rank of the group calls it."""
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

        ptrs = {"param": alloc(n * 4), "grad": alloc(n * 4), "flags": alloc(int(lib.dl_exchange_flag_bytes()))}
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
        self._own_ptrs = ptrs
        self._imported = []
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
                    self._imported.append(out.value)
            self._peer_ptrs[name] = arr
        # moments in the flat layout; a rank only ever touches its slices of them
        self.exp_avg = torch.zeros(n, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=dev)
        self._plan_exchange_buckets(buckets)
        self.state_t = torch.zeros((len(self._buckets), 16), dtype=torch.int32, device=dev)
        self._exchange = (rank, world)
        self._poll_limit = int(poll_limit)
        self._comm_stream = torch.cuda.Stream(device=dev)
        self._group = group
        self.exchange_enabled = True
        for p in self._params:
            p._dl_after_backward_w = self._gradient_launched
        self._begin_exchange_step()
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)
        return self

    def _plan_exchange_buckets(self, buckets):
        """Buckets of consecutive parameters: [(offset, count, [params])]; at most 32 (the library's flag words)."""
        order = sorted(self._params, key=lambda p: self._slices[p][0])
        n_buckets = len(order) if buckets is None else max(1, min(int(buckets), len(order)))
        n_buckets = min(n_buckets, 32)
        per = -(-len(order) // n_buckets)
        self._buckets, self._bucket_of = [], {}
        for bi in range(0, len(order), per):
            group = order[bi:bi + per]
            lo = self._slices[group[0]][0]
            last_off, last_cnt = self._slices[group[-1]]
            hi = last_off + (last_cnt + 3) // 4 * 4
            for p in group:
                self._bucket_of[p] = len(self._buckets)
            self._buckets.append((lo, hi - lo, group))

    def _begin_exchange_step(self):
        self._bucket_pending = [len(b[2]) for b in self._buckets]
        self._bucket_launched = [False] * len(self._buckets)

    def _gradient_launched(self, p):
        """Called by LogicLayer's backward right after the backward_w kernel of parameter `p` has been launched (on the
        current stream): when that completes a bucket, the bucket's exchange goes out."""
        bi = self._bucket_of.get(p)
        if bi is None or self._bucket_launched[bi]:
            return
        self._bucket_pending[bi] -= 1
        if self._bucket_pending[bi] <= 0:
            self._launch_bucket(bi)

    def _launch_bucket(self, bi):
        rank, world = self._exchange
        off, cnt, _ = self._buckets[bi]
        g = self.param_groups[0]
        beta1, beta2 = g['betas']
        lib = N.lib()
        dev = self.flat_param.device
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(dev))
        self._comm_stream.wait_event(ready)
        state = self.state_t[bi].data_ptr()
        with torch.cuda.device(dev):
            st = self._comm_stream.cuda_stream
            N.check(lib.dl_exchange_reduce_adam_f32(self._peer_ptrs["param"], self._peer_ptrs["grad"], self._peer_ptrs["flags"], rank,
                                                    world, self.exp_avg.data_ptr(), self.exp_avg_sq.data_ptr(), off, cnt, bi,
                                                    float(g['lr']), float(beta1), float(beta2), float(g['eps']), state,
                                                    self._poll_limit, st))
            N.check(lib.dl_exchange_gather_f32(self._peer_ptrs["param"], self._peer_ptrs["flags"], rank, world, off, cnt, bi, state,
                                               self._poll_limit, st))
        self._bucket_launched[bi] = True

    def exchange_error(self):
        """True when a wait for a peer ever ran out of its poll limit (synchronises).  The step in which that happened
        left parameters, moments and step count as they were; training cannot go on from there."""
        return bool(int(self.state_t[:, 2].max().item())) if getattr(self, "exchange_enabled", False) else False

    def exchange_timing(self):
        """Per bucket, nanoseconds inside the latest exchange on this rank (synchronises): waiting for all ranks'
        gradients, reduce + Adam on this rank's slice, from there to the gather kernel's start, waiting for all ranks'
        slices, fetching the other slices; `total_ns` from the reduce kernel's entry to the gather kernel's end."""
        if not getattr(self, "exchange_enabled", False):
            return None
        out = []
        for row in self.state_t[:, 4:16].cpu().contiguous().view(torch.int64).tolist():
            t = row
            out.append({"wait_gradients_ns": t[1] - t[0], "slice_ns": t[2] - t[1], "to_gather_ns": t[3] - t[2],
                        "wait_slices_ns": t[4] - t[3], "gather_ns": t[5] - t[4], "total_ns": t[5] - t[0], "entered_ns": t[0],
                        "done_ns": t[5]})
        return out

    def close(self):
        """Leaves the peer-memory exchange: the parameters move back into ordinary device memory, the peers' buffers are
        unmapped and this rank's are freed.  Collective in effect: call it on every rank, after the last step (a
        captured CUDA graph of the step must be dropped first -- TrainStep.close() does both)."""
        if not getattr(self, "exchange_enabled", False):
            return
        import torch.distributed as dist
        lib = N.lib()
        dev = self.flat_param.device
        torch.cuda.synchronize(dev)
        with torch.no_grad():
            keep_param = self.flat_param.clone()
            keep_grad = torch.zeros_like(keep_param)
            for p in self._params:
                off, cnt = self._slices[p]
                p.data = keep_param[off:off + cnt].view_as(p)
                p._dl_grad_out = keep_grad[off:off + cnt].view_as(p)
                p._dl_after_backward_w = None
                p.grad = None
        self.flat_param, self.flat_grad = keep_param, keep_grad
        self.exchange_enabled = False
        self.state_t = torch.zeros(2, dtype=torch.int32, device=dev)
        torch.cuda.synchronize(dev)
        try:
            dist.barrier(group=self._group)   # nobody unmaps or frees while a peer might still read
        except Exception:
            pass
        with torch.cuda.device(dev):
            for ptr in self._imported:
                N.check(lib.dl_comm_close(ptr))
            for ptr in self._own_ptrs.values():
                N.check(lib.dl_comm_free(ptr))
        self._imported, self._own_ptrs, self._peer_ptrs = [], {}, {}

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
            if getattr(self, "exchange_enabled", False):
                rank, world = self._exchange          # only this rank's slice of every bucket is touched
                for off, cnt, _ in self._buckets:
                    per = -(-(cnt // 4) // world) * 4
                    lo = off + min(rank * per, cnt)
                    nbytes = (min(lo + per, off + cnt) - lo) * 4
                    for t in (self.exp_avg, self.exp_avg_sq):
                        if nbytes > 0:
                            N.check(N.lib().dl_prefetch_l2(t.data_ptr() + lo * 4, nbytes, st))
                return
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
            # buckets whose gradients were not announced by a backward_w launch (none in a normal step) go out now;
            # then the current stream waits for the exchange
            for bi in range(len(self._buckets)):
                if not self._bucket_launched[bi]:
                    self._launch_bucket(bi)
            torch.cuda.current_stream(self.flat_param.device).wait_stream(self._comm_stream)
            self._begin_exchange_step()
            return loss
        with torch.cuda.device(self.flat_param.device):
            N.check(N.lib().dl_adam_step_f32(self.flat_param.data_ptr(), self.flat_grad.data_ptr(), self.exp_avg.data_ptr(),
                                             self.exp_avg_sq.data_ptr(), self.flat_param.numel(), float(g['lr']), float(beta1),
                                             float(beta2), float(g['eps']), float(self.grad_scale), self.state_t.data_ptr(),
                                             N.stream_of(self.flat_param)))
        return loss
