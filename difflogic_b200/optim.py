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


def plan_inboxes(bucket_counts, world):
    """Where each exchange bucket lies inside a sender's region of a packet inbox (dl_exchange_packets_f32).
    bucket_counts: floats per bucket (multiples of 4).  Returns (first float4 slot of every bucket, slots per region): a
    bucket takes ceil(float4 of the bucket / world) slots, the slice one rank owns."""
    offsets, slots = [], 0
    for count in bucket_counts:
        offsets.append(slots)
        slots += -(-(int(count) // 4) // int(world))
    return offsets, max(slots, 1)


class ExchangeUnavailable(RuntimeError):
    """enable_exchange could not map a peer's buffers; raised on EVERY rank of the group, with the optimizer untouched."""


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

    def enable_exchange(self, group=None, buckets=None, wait_limit_us=0, announce_in_backward=False, one_pass_bytes=8 << 20,
                        packet_bytes=2 << 20, push_in_backward=False):
        """Switches to the peer-memory exchange (dl_backward_w_announce_f32 / dl_exchange_bucket_f32): the flat
        parameter and gradient buffers move into memory that the other ranks of `group` (one process per GPU on this
        machine) map through CUDA IPC.  The buffers are cut into buckets -- one per parameter, or `buckets` groups of
        consecutive parameters.  A layer's backward_w kernel tells the peers when the bucket's gradients are complete,
        and the bucket's exchange kernel is launched right after it on a stream of its own: the gradients are averaged
        over the ranks, Adam is applied to this rank's slice, the new parameters are fetched from the other ranks, all
        beside the rest of the backward pass.  `step()` launches whatever is still missing and makes the current
        stream wait for the exchange.  No NCCL call is made per step.  Collective: every rank of the group calls it.
        Raises ExchangeUnavailable on every rank, with nothing changed, when a rank cannot map a peer's buffers.
        wait_limit_us: how long a kernel waits for the other ranks before it gives up (0: 20 seconds).
        announce_in_backward: the layer's backward_w kernel tells the peers that the gradients are complete (its last
        block does), instead of the exchange kernel at its start.
        one_pass_bytes: the buckets whose gradients come LAST in the backward pass -- the ones whose exchange little or
        nothing hides -- are exchanged in one pass (every rank averages and updates all of the bucket: one flag round
        trip less): as many buckets from the end as keep (ranks - 1) x their total size within this many bytes;
        0: never.
        packet_bytes: buckets of at most this many bytes are exchanged with the flags inside the data
        (dl_exchange_packets_f32: pushes only, no flag round trips, twice the bytes over NVLink); 0: none.
        push_in_backward: the backward_w kernel of a layer whose bucket goes as packets pushes the gradients itself, beside
        its arithmetic (dl_backward_w_push_f32), instead of the exchange kernel after it.  Off by default: the exchange
        kernel gets shorter, but the stores over NVLink stretch every backward_w kernel by more (config 2, two ranks:
        93.9 against 91.1 us per step)."""
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

        # the bucket plan first: the inboxes of the packet exchange have one region per sending rank with
        # ceil(bucket / ranks) float4 slots per bucket
        self._plan_exchange_buckets(buckets)
        self._inbox_off, self._inbox_stride = plan_inboxes([cnt for _, cnt, _ in self._buckets], world)
        self._packet_form = {bi for bi, (_, cnt, _) in enumerate(self._buckets) if world > 1 and 0 < cnt * 4 <= int(packet_bytes)}
        ptrs = {"param": alloc(n * 4), "grad": alloc(n * 4), "flags": alloc(int(lib.dl_exchange_flag_bytes()))}
        if self._packet_form:
            ptrs["grad_inbox"] = alloc(32 * world * self._inbox_stride)
            ptrs["param_inbox"] = alloc(32 * world * self._inbox_stride)
        handles = {}
        for name, ptr in ptrs.items():
            buf = (ctypes.c_ubyte * 64)()
            N.check(lib.dl_comm_export(ptr, buf))
            handles[name] = bytes(buf)
        gathered = [None] * world
        dist.all_gather_object(gathered, handles, group=group)
        # map the peers' buffers; a rank that cannot (no peer access between two of the GPUs) must not leave the others
        # waiting in the next collective, so the outcome is agreed on before anything of the optimizer has changed
        imported, peer_ptrs, failure = [], {}, None
        for name in ptrs:
            arr = (ctypes.c_void_p * world)()
            for r in range(world):
                if r == rank:
                    arr[r] = ptrs[name]
                    continue
                out = ctypes.c_void_p()
                with torch.cuda.device(dev):
                    rc = lib.dl_comm_import(gathered[r][name], ctypes.byref(out))
                if rc != 0:
                    failure = failure or "rank %d could not map the %s buffer of rank %d (%s)" % (rank, name, r, "status %d: %s" % (rc, N.last_error()))
                    continue
                arr[r] = out.value
                imported.append(out.value)
            peer_ptrs[name] = arr
        failures = [None] * world
        dist.all_gather_object(failures, failure, group=group)
        if any(failures):
            with torch.cuda.device(dev):
                for ptr in imported:
                    lib.dl_comm_close(ptr)
                for ptr in ptrs.values():
                    lib.dl_comm_free(ptr)
            raise ExchangeUnavailable("; ".join(f for f in failures if f))

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
        self._own_ptrs, self._imported, self._peer_ptrs = ptrs, imported, peer_ptrs
        # moments in the flat layout; a rank only ever touches its slices of them
        self.exp_avg = torch.zeros(n, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=dev)
        self.state_t = torch.zeros((len(self._buckets), 16), dtype=torch.int32, device=dev)
        self._bw_tickets = torch.zeros(len(self._params), dtype=torch.int32, device=dev)     # per parameter
        self._bucket_kernels = torch.zeros(len(self._buckets), dtype=torch.int32, device=dev)  # per bucket
        self._param_index = {p: i for i, p in enumerate(self._params)}
        self._exchange = (rank, world)
        self._barrier_state = None      # rank_barrier's own count, made on first use
        self._wait_limit_us = int(wait_limit_us)   # 0: the library's default (20 s); ranks further apart than that fail the step
        self._announce_in_backward = bool(announce_in_backward)
        self._one_pass_bytes = int(one_pass_bytes)
        self._push_in_backward = bool(push_in_backward)
        self._one_pass = set()          # buckets exchanged in one pass; fixed by the first step
        self._forms_fixed = False
        # a few streams for the buckets' exchange kernels, so that a bucket does not queue behind the one before it
        # (high priority: their few blocks are scheduled ahead of the backward kernels' many)
        self._comm_streams = [torch.cuda.Stream(device=dev, priority=-1) for _ in range(min(4, len(self._buckets)))]
        self._group = group
        self.exchange_enabled = True
        for p in self._params:
            p._dl_exchange = self
        self._begin_exchange_step()
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)
        return self

    def _plan_exchange_buckets(self, buckets):
        """Buckets of consecutive parameters: [(offset, count, [params])]; at most 31 (the library has flag words for 32;
        the last set is rank_barrier's)."""
        order = sorted(self._params, key=lambda p: self._slices[p][0])
        n_buckets = len(order) if buckets is None else max(1, min(int(buckets), len(order)))
        n_buckets = min(n_buckets, 31)
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
        self._bucket_done = []          # events: the buckets' exchange kernels of this step
        self._bucket_pushes = [0] * len(self._buckets)   # backward_w kernels of this step that pushed their gradients

    def backward_w(self, p, x, a, b, grad_y, grad_out, rows_per_class=1):
        """backward_w of the layer whose weights are `p`, called by LogicLayer's backward in place of the plain kernel:
        the kernel's last block tells the peers that this rank's gradients of p's bucket are complete, and once every
        backward_w of the bucket is in the queue the bucket's exchange kernel follows -- on a stream of its own,
        beside the rest of the backward pass; the bucket that comes last right behind its backward_w kernel."""
        from . import ops
        rank, world = self._exchange
        bi = self._bucket_of[p]
        if bi in self._packet_form and self._push_in_backward and grad_out is not None:
            # the kernel sends the other ranks' slices of its gradients into their inboxes while it is still computing
            off, cnt, _ = self._buckets[bi]
            out = ops.logic_backward_w_push(x, a, b, grad_y, p, grad_out, rows_per_class, self._peer_ptrs["grad_inbox"], rank, world,
                                            self._slices[p][0] - off, cnt, self._inbox_off[bi], self._inbox_stride, self.state_t[bi])
            self._bucket_pushes[bi] += 1
        elif self._announce_in_backward and bi not in self._packet_form:   # packets announce themselves
            out = ops.logic_backward_w_announce(x, a, b, grad_y, p, grad_out, rows_per_class, self._peer_ptrs["flags"], rank, world,
                                                bi, self.state_t[bi], self._bw_tickets[self._param_index[p]:],
                                                self._bucket_kernels[bi:], len(self._buckets[bi][2]))
        else:
            out = ops.logic_backward_w(x, a, b, grad_y, p, ops.W_LOGITS, out=grad_out, overlap=True, rows_per_class=rows_per_class)
        if not self._bucket_launched[bi]:
            self._bucket_pending[bi] -= 1
            if self._bucket_pending[bi] <= 0:
                last = sum(self._bucket_launched) == len(self._buckets) - 1
                if not self._forms_fixed:
                    # One pass for the buckets at the END of the backward pass, as many as fit the byte limit: this bucket
                    # and everything that is still to come.  (With two ranks that is every bucket: one pass then moves no
                    # more bytes than two.)
                    still = sum(b[1] for i, b in enumerate(self._buckets) if not self._bucket_launched[i])
                    if world > 1 and (world - 1) * still * 4 <= self._one_pass_bytes and bi not in self._packet_form:
                        self._one_pass.add(bi)
                    self._forms_fixed = last
                self._launch_bucket(bi, behind_backward_w=last, announce_here=not self._announce_in_backward)
        return out

    def _launch_bucket(self, bi, behind_backward_w, announce_here):
        rank, world = self._exchange
        off, cnt, _ = self._buckets[bi]
        g = self.param_groups[0]
        beta1, beta2 = g['betas']
        dev = self.flat_param.device
        current = torch.cuda.current_stream(dev)
        if behind_backward_w:
            stream = current     # the kernel's set-up overlaps the end of the backward_w kernel just before it
        else:
            stream = self._comm_streams[bi % len(self._comm_streams)]
            ready = torch.cuda.Event()
            ready.record(current)
            stream.wait_event(ready)
        how = N.LAUNCH_OVERLAP_SETUP if behind_backward_w else N.LAUNCH_PLAIN
        with torch.cuda.device(dev):
            if bi in self._packet_form:
                N.check(N.lib().dl_exchange_packets_f32(
                    self.flat_param.data_ptr(), self.flat_grad.data_ptr(), self._peer_ptrs["grad_inbox"], self._peer_ptrs["param_inbox"],
                    rank, world, self.exp_avg.data_ptr(), self.exp_avg_sq.data_ptr(), off, cnt, self._inbox_off[bi], self._inbox_stride,
                    float(g['lr']), float(beta1), float(beta2), float(g['eps']), self.state_t[bi].data_ptr(),
                    int(self._bucket_pushes[bi] == len(self._buckets[bi][2])),   # every backward_w of the bucket has pushed
                    self._wait_limit_us, how, stream.cuda_stream))
            else:
                N.check(N.lib().dl_exchange_bucket_f32(
                    self._peer_ptrs["param"], self._peer_ptrs["grad"], self._peer_ptrs["flags"], rank, world, self.exp_avg.data_ptr(),
                    self.exp_avg_sq.data_ptr(), off, cnt, bi, float(g['lr']), float(beta1), float(beta2), float(g['eps']),
                    self.state_t[bi].data_ptr(), int(announce_here), int(bi in self._one_pass), self._wait_limit_us, how,
                    stream.cuda_stream))
        done = torch.cuda.Event()
        done.record(stream)
        self._bucket_done.append(done)
        self._bucket_launched[bi] = True

    def rank_barrier(self):
        """Launches, on the current stream, a kernel in which the ranks of the exchange wait for each other (bounded like
        every wait of the exchange): what follows it on the stream starts at the same time on every rank, within a flag's
        latency.  No host synchronisation.  Collective: every rank launches it equally often."""
        rank, world = self._exchange
        if getattr(self, "_barrier_state", None) is None:
            self._barrier_state = torch.zeros(16, dtype=torch.int32, device=self.flat_param.device)
        with torch.cuda.device(self.flat_param.device):
            N.check(N.lib().dl_rank_barrier(self._peer_ptrs["flags"], rank, world, 31, self._barrier_state.data_ptr(),
                                            self._wait_limit_us, N.stream_of(self.flat_param)))

    def full_exp_avg(self):
        """Adam's first moments of ALL parameters in the flat layout.  Under the peer-memory exchange a rank holds the
        moments of its own slices only (of the whole bucket for one-pass buckets): they are put together with one
        all-reduce (collective; a diagnostic, not part of a step)."""
        if not getattr(self, "exchange_enabled", False):
            return self.exp_avg.detach().clone()
        import torch.distributed as dist
        rank, world = self._exchange
        m = self.exp_avg.detach().clone()
        if world > 1:
            for bi, (off, cnt, _) in enumerate(self._buckets):
                if bi in self._one_pass and rank != 0:
                    m[off:off + cnt] = 0        # every rank holds these in full: count them once
            dist.all_reduce(m, group=self._group)
        return m

    def exchange_error(self):
        """True when a wait for a peer ever ran out of its time limit (synchronises).  The step in which that happened
        left parameters, moments and step count as they were; training cannot go on from there."""
        if not getattr(self, "exchange_enabled", False):
            return False
        barrier = getattr(self, "_barrier_state", None)
        return bool(int(self.state_t[:, 2].max().item())) or (barrier is not None and bool(int(barrier[2].item())))

    def exchange_timing(self):
        """Per bucket, nanoseconds inside the latest exchange on this rank (synchronises): waiting for all ranks'
        gradients, reduce + Adam on this rank's slice, waiting for all ranks' slices, fetching the other slices;
        `total_ns` from the kernel's entry to its end.  For a bucket exchanged as packets the four spans are, on the
        kernel's first block: pushing the gradients, reducing the own slice as the packets arrive, [nothing], taking the
        other slices' parameters out of the inbox -- then until the last block is through."""
        if not getattr(self, "exchange_enabled", False):
            return None
        out = []
        for bi, row in enumerate(self.state_t[:, 4:16].cpu().contiguous().view(torch.int64).tolist()):
            t = row
            out.append({"form": "packets" if bi in self._packet_form else "one pass" if bi in self._one_pass else "two passes",
                        "wait_gradients_ns": t[1] - t[0], "slice_ns": t[2] - t[1], "wait_slices_ns": t[4] - t[2],
                        "gather_ns": t[5] - t[4], "total_ns": t[5] - t[0], "entered_ns": t[0], "done_ns": t[5],
                        "stamps_ns": [t[0], t[1], t[2], t[4], t[5]]})
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
                p._dl_exchange = None
                p.grad = None
        self.flat_param, self.flat_grad = keep_param, keep_grad
        self.exchange_enabled = False
        self._barrier_state = None
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
                return   # a rank touches only its slices, and the exchange kernels read them beside their peer loads
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
            # buckets whose exchange did not go out from a backward_w launch (gradients that came from elsewhere; none in
            # a normal step) go out now and announce themselves; then the current stream waits for every bucket
            for bi in range(len(self._buckets)):
                if not self._bucket_launched[bi]:
                    self._bucket_kernels[bi:bi + 1].zero_()
                    self._launch_bucket(bi, behind_backward_w=False, announce_here=True)
            self._forms_fixed = True
            current = torch.cuda.current_stream(self.flat_param.device)
            for done in self._bucket_done:
                current.wait_event(done)
            self._begin_exchange_step()
            return loss
        with torch.cuda.device(self.flat_param.device):
            N.check(N.lib().dl_adam_step_f32(self.flat_param.data_ptr(), self.flat_grad.data_ptr(), self.exp_avg.data_ptr(),
                                             self.exp_avg_sq.data_ptr(), self.flat_param.numel(), float(g['lr']), float(beta1),
                                             float(beta2), float(g['eps']), float(self.grad_scale), self.state_t.data_ptr(),
                                             N.stream_of(self.flat_param)))
        return loss
