"""Training step of a logic gate network: eager or captured in a CUDA graph, on one GPU or
batch-sharded over several (one process per GPU).

The reference has no multi-GPU code; its step is `loss_fn(model(x), y) -> zero_grad -> backward ->
optimizer.step` (experiments/main.py:174-181).  `TrainStep` runs exactly that.  When a process
group is given, every rank holds a full replica of the weights and connection indices, works on
its own shard of the batch, and only the `[out_dim, 16]` weight gradients are averaged over the
ranks: by FlatAdam's peer-memory exchange (two small kernels per layer, launched on a stream of
their own as soon as the layer's backward_w is in the queue) or by NCCL all-reduces on a side
stream, launched as soon as the gradients of a bucket of layers have been written; either way
the exchange overlaps the rest of the backward pass.  Nothing else crosses GPUs.

`capture()` records the whole step (H2D staging excluded) in one CUDA graph: the model's kernels
launch on torch's current stream, allocate nothing themselves and never synchronise, so a step of
~25 small kernels replays without per-launch host overhead.
"""
import torch
import torch.distributed as dist


class TrainStep:
    def __init__(self, model, optimizer, loss_fn=None, process_group=None, world_size=None, buckets=2, fuse_head=True,
                 step_in_backward=True):
        """
        :param model:         module on the current CUDA device (replicated on every rank)
        :param optimizer:     its optimizer; for `capture()` it must be graph-capturable
                              (difflogic_b200.optim.FlatAdam, or torch.optim.Adam(..., capturable=True))
        :param loss_fn:       defaults to CrossEntropyLoss (mean over the local batch)
        :param process_group: torch.distributed group to average gradients over, or None
        :param fuse_head:     when the model ends in GroupSum and the loss is a default CrossEntropyLoss, run the two
                              as one autograd node (same numbers, three kernels instead of five).  The fused
                              kernels take class-index targets in [0, k) only: they have no `ignore_index`
                              (torch's default -100 included), and a target outside the range would count as
                              "no class".  The targets of the first eager step are checked, once, on the host.
        :param step_in_backward: single GPU, FlatAdam, every parameter a CUDA LogicLayer's weights: the Adam update runs
                              in the epilogue of each layer's backward_w kernel instead of a kernel of its own after
                              the backward pass (same numbers; `.grad` is then not populated)
        :param buckets:       with FlatAdam: number of contiguous pieces of the flat gradient buffer that are
                              all-reduced separately (the piece holding the last layers first); 1 = one
                              all-reduce after the whole backward pass.  Other optimizers: one per parameter.
        """
        self.model = model
        self.optimizer = optimizer
        self.loss_fn = loss_fn if loss_fn is not None else torch.nn.CrossEntropyLoss()
        self.group = process_group
        self.world_size = world_size if world_size is not None else (
            dist.get_world_size(process_group) if process_group is not None else 1)
        self.params = [p for p in model.parameters() if p.requires_grad]
        self._graph = None
        self._resident = []
        self._static_x = self._static_y = self._static_loss = None
        self._comm_stream = None
        self._bw_stream = torch.cuda.Stream() if all(p.is_cuda for p in self.params) else None
        self._hooks = []
        self._on_gpu = all(p.is_cuda for p in self.params)
        self._bucket_of = {}       # param -> bucket index
        self._bucket_slices = []   # flat gradient slice of each bucket
        self._bucket_sizes = []    # parameters per bucket
        self._pending = []
        # FlatAdam.enable_exchange(): the optimizer launches the exchange itself, from the layers' backward
        self._exchange_in_optimizer = bool(getattr(optimizer, "exchange_enabled", False))
        self._body = self._head = self._pre = self._last = None
        self._unit_grad = None     # gradient of the loss w.r.t. itself, made once (autograd would fill a new one per step)
        if fuse_head and self._on_gpu and self._head_is_fusable(model, self.loss_fn):
            self._body, self._head = model[:-1], model[-1]
            from .difflogic import LogicLayer
            last = self._body[-1] if len(self._body) > 0 else None
            if isinstance(last, LogicLayer) and getattr(last, "implementation", None) == "cuda":
                self._pre, self._last = self._body[:-1], last   # everything before the last logic layer, and that layer
        self._targets_checked = False
        self._in_backward = False
        if (step_in_backward and self._on_gpu and self.world_size == 1 and not self._exchange_in_optimizer
                and hasattr(optimizer, "enable_step_in_backward") and self._all_logic_weights(model, optimizer)):
            self._in_backward = True   # switched on around each backward pass only: outside a step the model is as usual
            optimizer.enable_step_in_backward(True)    # allocates the per-layer step counts
            optimizer.enable_step_in_backward(False)
            optimizer.sync_step_counts(to_layers=True)
        if self.group is not None and self.world_size > 1 and not self._exchange_in_optimizer:
            if self._on_gpu:
                self._comm_stream = torch.cuda.Stream()
                self._plan_buckets(max(1, int(buckets)))
            for p in self.params:
                self._hooks.append(p.register_post_accumulate_grad_hook(self._reduce_when_ready))

    @staticmethod
    def _all_logic_weights(model, optimizer):
        """True when the optimizer's parameters are exactly the weights of the model's CUDA LogicLayers."""
        from .difflogic import LogicLayer
        mine = {id(m.weights) for m in model.modules() if isinstance(m, LogicLayer) and m.implementation == "cuda"}
        theirs = [p for g in optimizer.param_groups for p in g["params"]]
        return len(theirs) > 0 and all(id(p) in mine for p in theirs)

    @staticmethod
    def _head_is_fusable(model, loss_fn):
        from .difflogic import GroupSum
        from .losses import CrossEntropyLoss
        if not (isinstance(model, torch.nn.Sequential) and len(model) >= 2 and isinstance(model[-1], GroupSum)):
            return False
        if isinstance(loss_fn, CrossEntropyLoss):
            return True
        return (type(loss_fn) is torch.nn.CrossEntropyLoss and loss_fn.weight is None and loss_fn.reduction == "mean"
                and loss_fn.ignore_index == -100 and loss_fn.label_smoothing == 0.0)

    def _check_targets_once(self, y):
        """The fused head has no ignore_index: the first batch of targets that is seen outside a graph capture must
        lie in [0, k) (one host synchronisation, once)."""
        if self._targets_checked or not y.is_cuda or torch.cuda.is_current_stream_capturing():
            return
        self._targets_checked = True
        k = int(self._head.k)
        if y.numel() and (int(y.min()) < 0 or int(y.max()) >= k):
            raise ValueError("TrainStep: targets must be class indices in [0, %d); the fused GroupSum + cross-entropy head "
                             "implements no ignore_index (pass fuse_head=False to use the loss module as it is)" % k)

    def _loss(self, x, y):
        if self._head is not None:
            self._check_targets_once(y)
            if self._last is not None:
                # last layer + GroupSum + loss as one autograd node
                from .difflogic import logic_layer_head
                h = self._pre(x)
                out = logic_layer_head(self._last, h, y, self._head.k, float(self._head.tau)) if h.dim() == 2 else None
                if out is not None:
                    return out[0]
                h = self._last(h)
            else:
                h = self._body(x)
            if h.is_cuda and h.dtype == torch.float32 and h.dim() == 2 and y.dtype == torch.int64 and y.dim() == 1:
                from .losses import group_sum_cross_entropy
                return group_sum_cross_entropy(h, y, self._head.k, float(self._head.tau))[0]
            return self.loss_fn(self._head(h), y)
        return self.loss_fn(self.model(x), y)

    # -- gradient exchange -----------------------------------------------------------------------

    def _plan_buckets(self, n_buckets):
        """With a flat gradient buffer (FlatAdam), groups consecutive parameters into `n_buckets` slices of it."""
        slices = getattr(self.optimizer, "_slices", None)
        flat = getattr(self.optimizer, "flat_grad", None)
        if slices is None or flat is None or any(p not in slices for p in self.params):
            return
        order = sorted(self.params, key=lambda p: slices[p][0])
        n_buckets = min(n_buckets, len(order))
        per = -(-len(order) // n_buckets)
        for bi in range(n_buckets):
            group = order[bi * per:(bi + 1) * per]
            if not group:
                continue
            lo = slices[group[0]][0]
            hi = slices[group[-1]][0] + slices[group[-1]][1]
            for p in group:
                self._bucket_of[p] = len(self._bucket_slices)
            self._bucket_slices.append(flat[lo:hi])
            self._bucket_sizes.append(len(group))
        self._pending = list(self._bucket_sizes)

    def _launch_all_reduce(self, tensor):
        main = torch.cuda.current_stream()
        ready = torch.cuda.Event()
        ready.record(main)
        self._comm_stream.wait_event(ready)
        with torch.cuda.stream(self._comm_stream):
            dist.all_reduce(tensor, op=dist.ReduceOp.AVG, group=self.group)

    def _reduce_when_ready(self, param):
        """Runs right after `param.grad` has been written by the layer's backward_w."""
        if not self._on_gpu:
            # host tensors (the pure-python implementation, gloo): no streams, and gloo has no AVG
            dist.all_reduce(param.grad, op=dist.ReduceOp.SUM, group=self.group)
            param.grad.div_(self.world_size)
            return
        if param in self._bucket_of:
            bi = self._bucket_of[param]
            self._pending[bi] -= 1
            if self._pending[bi] == 0:
                self._launch_all_reduce(self._bucket_slices[bi])
            return
        self._launch_all_reduce(param.grad)

    def _join_comm(self):
        if self._comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self._comm_stream)

    # -- the step --------------------------------------------------------------------------------

    def _step(self, x, y):
        from . import difflogic as _dl
        self._pending = list(self._bucket_sizes)
        loss = self._loss(x, y)
        self.optimizer.zero_grad(set_to_none=True)
        if self._on_gpu and (self._unit_grad is None or self._unit_grad.device != loss.device):
            self._unit_grad = torch.ones((), dtype=loss.dtype, device=loss.device)
            self._unit_grad._dl_is_one = True   # lets the fused head skip the multiplication by the incoming gradient
        # backward_w of every layer runs on a side stream, off the chain of backward_x kernels -- unless gradient
        # hooks (the NCCL path) need the gradients in stream order
        side = self._bw_stream if (self._on_gpu and not self._hooks) else None
        if side is not None:
            _dl.set_backward_w_stream(side)
            if hasattr(self.optimizer, "prefetch_state") and not self._in_backward:
                # warm the optimizer's moments in L2 beside the backward pass
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    self.optimizer.prefetch_state()
        if self._in_backward:
            self.optimizer.enable_step_in_backward(True)
        try:
            loss.backward(gradient=self._unit_grad if self._on_gpu else None)
        finally:
            if self._in_backward:
                self.optimizer.enable_step_in_backward(False)
            if side is not None:
                _dl.set_backward_w_stream(None)
                torch.cuda.current_stream().wait_stream(side)
        self._join_comm()
        if not self._in_backward:    # else the backward_w kernels have applied the update
            self.optimizer.step()
        return loss.detach()

    def __call__(self, x, y):
        """One step on device tensors; returns the (local) loss as a device scalar."""
        if self._graph is None:
            return self._step(x, y)
        self._static_x.copy_(x, non_blocking=True)
        self._static_y.copy_(y, non_blocking=True)
        self._graph.replay()
        return self._static_loss

    def capture(self, x, y, warmup=3):
        """Captures the step in a CUDA graph.  `x`, `y` give the shapes; their contents are used for
        `warmup` eager steps (they DO update the weights) that run before the capture."""
        self._static_x = x.clone()
        self._static_y = y.clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self._step(self._static_x, self._static_y)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._static_loss = self._step(self._static_x, self._static_y)
        self._graph = graph
        return self

    def capture_resident(self, xs, ys):
        """After capture(): one more graph per batch (xs[i], ys[i]) that reads its inputs where they ARE -- device tensors
        that stay alive and in place -- instead of the static buffers, for batches that are already resident in device
        memory (no copy into the static buffers in front of a step).  The graphs share the first graph's memory pool.
        Returns the number of graphs; replay_resident(i) runs the step on batch i."""
        if self._graph is None:
            raise RuntimeError("TrainStep.capture_resident: call capture() first")
        self._resident = []
        for x, y in zip(xs, ys):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, pool=self._graph.pool()):
                loss = self._step(x, y)
            self._resident.append((graph, loss, x, y))
        return len(self._resident)

    def replay_resident(self, i):
        """Replays the step captured on resident batch i (whatever that batch's tensors hold now)."""
        graph, loss = self._resident[i][0], self._resident[i][1]
        graph.replay()
        return loss

    @property
    def static_inputs(self):
        return self._static_x, self._static_y

    def replay(self):
        """Replays the captured step on whatever the static input buffers hold."""
        self._graph.replay()
        return self._static_loss

    def close(self):
        """Drops the captured graph and the gradient hooks.  Call it before tearing down the process group: a
        graph that holds captured collectives must not outlive the communicator."""
        for h in self._hooks:
            h.remove()
        self._hooks = []
        if self._in_backward:
            self.optimizer.sync_step_counts(to_layers=False)   # optimizer.step() can take over from here
        self._in_backward = False
        if self._on_gpu and torch.cuda.is_available():
            torch.cuda.synchronize()
        self._graph = None
        self._static_loss = None
        self._resident = []
        if self._exchange_in_optimizer and hasattr(self.optimizer, "close"):
            self.optimizer.close()   # unmaps the peers' buffers; the parameters move back to ordinary memory
            self._exchange_in_optimizer = False


def shard_range(n_samples, rank, world_size, multiple=1):
    """[start, stop) of the samples rank `rank` works on when `n_samples` are split over `world_size` ranks in
    contiguous pieces whose sizes are multiples of `multiple` (64 for packed int64 words: a shard is then a
    column range of whole words of the packed tensor); the last rank takes the remainder."""
    units = -(-n_samples // multiple)
    per = -(-units // world_size)
    start = min(rank * per * multiple, n_samples)
    stop = min((rank + 1) * per * multiple, n_samples)
    return start, stop
