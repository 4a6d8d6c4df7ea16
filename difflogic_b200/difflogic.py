"""LogicLayer and GroupSum on the B200 kernels.

Drop-in for the reference module difflogic/difflogic.py (constructor arguments, attributes,
method names, tensor layouts and error behaviour are kept).  With `implementation='cuda'` every
layer runs on the library declared in include/difflogic_b200.h:

* training / float eval:  one forward kernel that takes the raw `weights` (softmax or arg-max is
  done inside it), `backward_w` with the softmax backward folded in, `backward_x` through a
  pre-built gather plan with `grad_factor` folded in;
* PackBitsTensor input:   the packed-bit eval kernel;
* GroupSum:               a feature-major reduction kernel (float) or the group bit-sum (packed).

`implementation='python'` is the pure-torch definition of the same layer and runs anywhere.
"""
import torch

from . import ops
from .functional import GradFactor, bin_op_s, get_unique_connections
from .packbitstensor import PackBitsTensor


# Optional side stream for backward_w.  Inside one layer, backward_x (which the next layer's backward waits for)
# and backward_w (which only the optimizer waits for) are independent; with a side stream set, backward_w leaves
# the critical path of the backward pass.  Whoever sets it must make the main stream wait for it before the
# gradients are used (difflogic_b200.training.TrainStep does both).
_backward_w_stream = None


# DIFFLOGIC_DEBUG=1: every CUDA LogicLayer checks its index tensors on the device when they are set (the kernels trust
# them afterwards); read once, at import.
import os as _os
_DEBUG_CHECKS = _os.environ.get("DIFFLOGIC_DEBUG", "0") == "1"


def set_backward_w_stream(stream):
    """Sets (or, with None, clears) the CUDA stream on which LogicLayer's backward_w kernels are launched."""
    global _backward_w_stream
    _backward_w_stream = stream


def _is_cuda_device(device):
    try:
        return torch.device(device).type == 'cuda'
    except (RuntimeError, TypeError):
        return False


class LogicLayer(torch.nn.Module):
    """A layer of `out_dim` two-input logic gates, each a learned mix of the 16 possible gates."""

    def __init__(
            self,
            in_dim: int,
            out_dim: int,
            device: str = 'cuda',
            grad_factor: float = 1.,
            implementation: str = None,
            connections: str = 'random',
    ):
        """
        :param in_dim:         number of input features
        :param out_dim:        number of gates (= output features)
        :param device:         'cuda' or 'cpu'
        :param grad_factor:    scales the gradient flowing to the layer input (use e.g. 2 for nets deeper than ~6)
        :param implementation: 'cuda' (the kernels; default on a CUDA device) or 'python' (pure torch; default on CPU)
        :param connections:    'random' or 'unique'
        """
        super().__init__()
        self.weights = torch.nn.parameter.Parameter(torch.randn(out_dim, 16, device=device))
        self.in_dim = in_dim
        self.out_dim = out_dim
        self.device = device
        self.grad_factor = grad_factor

        self.implementation = implementation
        if self.implementation is None:
            self.implementation = 'cuda' if _is_cuda_device(device) else 'python'
        assert self.implementation in ['cuda', 'python'], self.implementation

        self.connections = connections
        assert self.connections in ['random', 'unique'], self.connections
        self.indices = self.get_connections(self.connections, device)

        if self.implementation == 'cuda':
            self._build_inverse_index()

        self.num_neurons = out_dim
        self.num_weights = out_dim

    # -- connection set-up ---------------------------------------------------------------------------------------

    def get_connections(self, connections, device='cuda'):
        assert self.out_dim * 2 >= self.in_dim, 'The number of neurons ({}) must not be smaller than half of the ' \
                                                'number of inputs ({}) because otherwise not all inputs could be ' \
                                                'used or considered.'.format(self.out_dim, self.in_dim)
        if connections == 'random':
            # every input is used floor/ceil(2*out/in) times; both draws come from the CPU generator
            slots = torch.randperm(2 * self.out_dim) % self.in_dim
            slots = torch.randperm(self.in_dim)[slots]
            a, b = slots.reshape(2, self.out_dim).to(torch.int64).to(device)
            return a, b
        elif connections == 'unique':
            return get_unique_connections(self.in_dim, self.out_dim, device)
        else:
            raise ValueError(connections)

    def _build_inverse_index(self):
        """Inverse connection index used by backward_x.

        `given_x_indices_of_y_start` / `given_x_indices_of_y` have the reference's meaning
        (difflogic.py:56-69); `_plan` is the same index with the partner row and the input slot
        resolved, which is what the kernel walks."""
        a, b = self.indices
        self.indices = (a.contiguous(), b.contiguous())
        a, b = self.indices
        self.given_x_indices_of_y_start, self.given_x_indices_of_y = ops.inverse_index(a, b, self.in_dim)
        if a.is_cuda:
            if _DEBUG_CHECKS:
                ops.check_connections(a, b, self.in_dim)      # before anything is computed from them
            self._plan = ops.build_backward_plan(a, b, self.given_x_indices_of_y_start, self.given_x_indices_of_y)
            if _DEBUG_CHECKS:
                ops.check_connections(a, b, self.in_dim, self.given_x_indices_of_y_start, self.given_x_indices_of_y, self._plan)
            # the layer's kernels may read these index tensors ahead of the kernel that precedes them in the
            # stream (DL_LAUNCH_OVERLAP_SETUP), so they must be final before any such launch is queued
            torch.cuda.current_stream(a.device).synchronize()
        else:
            self._plan = None

    def set_connections(self, a, b):
        """Replaces the connection indices (e.g. to copy them from another model) and rebuilds the inverse index."""
        assert a.shape == (self.out_dim,) and b.shape == (self.out_dim,), (a.shape, b.shape)
        dev = self.weights.device
        self.indices = (a.to(dev, torch.int64).contiguous(), b.to(dev, torch.int64).contiguous())
        if self.implementation == 'cuda':
            self._build_inverse_index()

    def _apply(self, fn, *args, **kwargs):
        # indices are plain attributes (not buffers), as in the reference; keep them on the weights' device
        super()._apply(fn, *args, **kwargs)
        dev = self.weights.device
        if self.indices[0].device != dev:
            self.indices = (self.indices[0].to(dev), self.indices[1].to(dev))
            if self.implementation == 'cuda':
                self._build_inverse_index()
        return self

    # -- forward -------------------------------------------------------------------------------------------------

    def forward(self, x):
        if isinstance(x, PackBitsTensor):
            assert not self.training, 'PackBitsTensor is not supported for the differentiable training mode.'
            assert _is_cuda_device(self.device), 'PackBitsTensor is only supported for CUDA, not for {}. ' \
                                                 'If you want fast inference on CPU, please use CompiledDiffLogicModel.' \
                                                 ''.format(self.device)
            if self.implementation == 'cuda':
                return self.forward_cuda_eval(x)
            raise ValueError(self.implementation)

        if self.implementation == 'cuda':
            return self.forward_cuda(x)  # grad_factor is applied inside backward_x
        elif self.implementation == 'python':
            if self.grad_factor != 1.:
                x = GradFactor.apply(x, self.grad_factor)
            return self.forward_python(x)
        else:
            raise ValueError(self.implementation)

    def forward_python(self, x):
        assert x.shape[-1] == self.in_dim, (x[0].shape[-1], self.in_dim)
        a, b = x[..., self.indices[0]], x[..., self.indices[1]]
        if self.training:
            mix = torch.nn.functional.softmax(self.weights, dim=-1)
        else:
            mix = torch.nn.functional.one_hot(self.weights.argmax(-1), 16).to(torch.float32)
        return bin_op_s(a, b, mix)

    def forward_cuda(self, x):
        if self.training:
            assert x.device.type == 'cuda', x.device
        assert x.ndim == 2, x.ndim

        # feature-major: a no-op after another LogicLayer; the network's input goes through the library's transpose
        xt = x.transpose(0, 1)
        if (not xt.is_contiguous() and x.is_contiguous() and x.is_cuda and x.dtype == torch.float32
                and not (x.requires_grad and torch.is_grad_enabled())):
            x = ops.transpose(x)
        else:
            x = xt.contiguous()
        assert x.shape[0] == self.in_dim, (x.shape, self.in_dim)
        if self._plan is None:
            raise RuntimeError('LogicLayer(implementation="cuda") needs its weights on a CUDA device')

        a, b = self.indices
        if self.training:
            y = LogicLayerFunction.apply(x, self.weights, a, b, self.given_x_indices_of_y_start, self._plan,
                                         float(self.grad_factor), getattr(self.weights, '_dl_grad_out', None))
        else:
            with torch.no_grad():
                y, _ = ops.logic_forward(x, a, b, self.weights, ops.W_ARGMAX, overlap=True)
        return y.transpose(0, 1)

    def forward_cuda_eval(self, x: PackBitsTensor):
        """
        WARNING: this is an in-place operation on `x` (its `.t` is replaced by this layer's output).
        """
        assert not self.training
        assert isinstance(x, PackBitsTensor)
        x._push_layer(self)  # evaluated when x.t is read, or fused with the other layers by GroupSum
        return x

    def _gate_ids(self):
        """uint8 arg-max gate per neuron, cached until the weights change."""
        w = self.weights
        key = (w.data_ptr(), w._version)
        cached = getattr(self, '_gate_cache', None)
        if cached is None or cached[0] != key:
            with torch.no_grad():
                cached = (key, ops.argmax_gates(w.detach().contiguous()))
            self._gate_cache = cached
        return cached[1]

    def extra_repr(self):
        return '{}, {}, {}'.format(self.in_dim, self.out_dim, 'train' if self.training else 'eval')


########################################################################################################################


class GroupSum(torch.nn.Module):
    """Sums the outputs in k groups and divides by tau (float input) or counts set bits per group (packed input)."""

    def __init__(self, k: int, tau: float = 1., device='cuda'):
        """
        :param k:      number of groups, e.g. the number of classes
        :param tau:    softmax temperature; float sums are divided by it (packed counts are not)
        :param device:
        """
        super().__init__()
        self.k = k
        self.tau = tau
        self.device = device

    def forward(self, x):
        if isinstance(x, PackBitsTensor):
            return x.group_sum(self.k)

        assert x.shape[-1] % self.k == 0, (x.shape, self.k)
        if x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and x.shape[0] > 0:
            return GroupSumFunction.apply(x, self.k, float(self.tau))
        return x.reshape(*x.shape[:-1], self.k, x.shape[-1] // self.k).sum(-1) / self.tau

    def extra_repr(self):
        return 'k={}, tau={}'.format(self.k, self.tau)


########################################################################################################################


def _run_backward_w(x, a, b, grad, weights, grad_out, rows_per_class=1):
    """backward_w of a layer; with an optimizer that steps inside backward (FlatAdam.enable_step_in_backward) the
    weights are updated by the same kernel and there is no gradient to return."""
    opt = getattr(weights, '_dl_adam', None)
    if opt is not None:
        ops.logic_backward_w_adam(x, a, b, grad, weights.data, overlap=True, rows_per_class=rows_per_class,
                                  **opt.backward_args(weights))
        return None
    exchange = getattr(weights, '_dl_exchange', None)
    if exchange is not None:
        # FlatAdam's peer-memory exchange: the kernel announces the gradient to the peers, the layer's exchange follows
        return exchange.backward_w(weights, x, a, b, grad, grad_out, rows_per_class)
    return ops.logic_backward_w(x, a, b, grad, weights, ops.W_LOGITS, out=grad_out, overlap=True, rows_per_class=rows_per_class)


class LogicLayerFunction(torch.autograd.Function):
    """Autograd node of one logic layer on feature-major tensors, from the raw weights.

    Replaces the reference's LogicLayerCudaFunction (difflogic.py:205-221) together with the softmax
    in front of it and the GradFactor node before the layer."""

    @staticmethod
    def forward(ctx, x, weights, a, b, start, plan, grad_factor, grad_out=None):
        y, coef = ops.logic_forward(x, a, b, weights, ops.W_LOGITS, want_coef=True, overlap=True)
        ctx.save_for_backward(x, weights, a, b, start, plan, coef)
        ctx.grad_factor = grad_factor
        ctx.grad_out = grad_out  # optional [out_dim, 16] buffer (a slice of a flat gradient bucket) for backward_w
        return y

    @staticmethod
    def backward(ctx, grad_y):
        x, weights, a, b, start, plan, coef = ctx.saved_tensors
        grad_y = grad_y.contiguous()
        grad_x = grad_w = None
        side = _backward_w_stream if (ctx.needs_input_grad[0] and ctx.needs_input_grad[1]) else None
        if side is not None:
            # fork: backward_w on the side stream, backward_x stays on the stream the next layer is waiting on
            main = torch.cuda.current_stream(x.device)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                grad_w = _run_backward_w(x, a, b, grad_y, weights, ctx.grad_out)
            for t in (x, grad_y, weights):
                t.record_stream(side)
            grad_x = ops.logic_backward_x(x, coef, grad_y, start, plan, ctx.grad_factor, overlap=True)
        else:
            if ctx.needs_input_grad[0]:
                grad_x = ops.logic_backward_x(x, coef, grad_y, start, plan, ctx.grad_factor, overlap=True)
            if ctx.needs_input_grad[1]:
                grad_w = _run_backward_w(x, a, b, grad_y, weights, ctx.grad_out)
        if grad_w is not None and ctx.grad_out is not None:
            # a fresh alias that nothing else references: autograd then adopts it as `weights.grad`
            # instead of copying it, so the gradient stays inside the flat bucket
            grad_w = grad_w.view(grad_w.shape)
        return grad_x, grad_w, None, None, None, None, None, None


class LogicLayerHeadFunction(torch.autograd.Function):
    """The LAST logic layer, GroupSum and the mean cross-entropy loss as one autograd node (training).

    forward : the layer's forward kernel adds up its rows per class and CTA (the output itself is never stored), then one
              small kernel finishes the class sums and computes the loss and the gradient of the loss w.r.t. the class
              scores (ops.logic_forward_head); sizes outside that path: layer forward, then ops.groupsum_cross_entropy;
    backward: the layer's backward_w / backward_x read that gradient as "one row per class" -- the `[n, batch]`
              gradient of the layer's output, whose rows are equal within a class, is never formed.
    Replaces LogicLayerFunction -> GroupSumFunction -> CrossEntropyLoss for the tail of
    `loss_fn(model(x), y)` (experiments/main.py:175) with the same numbers."""

    @staticmethod
    def forward(ctx, x, weights, a, b, start, plan, grad_factor, grad_out, target, k, tau):
        n_out = weights.shape[0]
        if ops.forward_head_applicable(n_out, x.shape[1], k):
            # the layer's rows are added up per class inside the forward kernel; its output is never stored
            loss, scores, grad_classes, coef = ops.logic_forward_head(x, a, b, weights, target, k, tau)
        else:
            y, coef = ops.logic_forward(x, a, b, weights, ops.W_LOGITS, want_coef=True, overlap=True)
            loss, scores, grad_classes = ops.groupsum_cross_entropy(y, target, k, tau)
        ctx.save_for_backward(x, weights, a, b, start, plan, coef, grad_classes)
        ctx.grad_factor, ctx.grad_out, ctx.rows_per_class = grad_factor, grad_out, n_out // k
        ctx.mark_non_differentiable(scores)
        ctx.set_materialize_grads(False)
        return loss, scores

    @staticmethod
    def backward(ctx, grad_loss, _grad_scores):
        if grad_loss is None:
            return (None,) * 11
        x, weights, a, b, start, plan, coef, grad_classes = ctx.saved_tensors
        if not getattr(grad_loss, '_dl_is_one', False):
            grad_classes = grad_classes * grad_loss     # a gradient other than the marked unit tensor: scale (one more kernel)
        m = ctx.rows_per_class
        grad_x = grad_w = None
        side = _backward_w_stream if (ctx.needs_input_grad[0] and ctx.needs_input_grad[1]) else None
        if side is not None:
            main = torch.cuda.current_stream(x.device)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                grad_w = _run_backward_w(x, a, b, grad_classes, weights, ctx.grad_out, rows_per_class=m)
            for t in (x, grad_classes, weights):
                t.record_stream(side)
            grad_x = ops.logic_backward_x(x, coef, grad_classes, start, plan, ctx.grad_factor, overlap=True, rows_per_class=m)
        else:
            if ctx.needs_input_grad[0]:
                grad_x = ops.logic_backward_x(x, coef, grad_classes, start, plan, ctx.grad_factor, overlap=True, rows_per_class=m)
            if ctx.needs_input_grad[1]:
                grad_w = _run_backward_w(x, a, b, grad_classes, weights, ctx.grad_out, rows_per_class=m)
        if grad_w is not None and ctx.grad_out is not None:
            grad_w = grad_w.view(grad_w.shape)  # a fresh alias: autograd adopts it as `weights.grad` without copying
        return (grad_x, grad_w) + (None,) * 9


def logic_layer_head(layer, x, target, k, tau):
    """(loss, scores) of `CrossEntropyLoss()(GroupSum(k, tau)(layer(x)), target)` for a CUDA LogicLayer in training mode
    and `x` of shape `[batch, in_dim]`; None when the fused kernel does not take the sizes (the caller then runs the
    three modules)."""
    if not (layer.training and layer._plan is not None and x.is_cuda and x.dtype == torch.float32 and x.dim() == 2
            and target.dtype == torch.int64 and target.dim() == 1 and layer.out_dim % k == 0
            and (ops.groupsum_cross_entropy_applicable(layer.out_dim, x.shape[0], k)
                 or ops.forward_head_applicable(layer.out_dim, x.shape[0], k))):
        return None
    xt = x.transpose(0, 1).contiguous()
    a, b = layer.indices
    return LogicLayerHeadFunction.apply(xt, layer.weights, a, b, layer.given_x_indices_of_y_start, layer._plan,
                                        float(layer.grad_factor), getattr(layer.weights, '_dl_grad_out', None),
                                        target.contiguous(), int(k), float(tau))


class LogicLayerCudaFunction(torch.autograd.Function):
    """The reference's autograd node with its exact signature (difflogic.py:205-221): `w` holds mixing
    weights that are already soft-maxed, and the result is the gradient w.r.t. those."""

    @staticmethod
    def forward(ctx, x, a, b, w, given_x_indices_of_y_start, given_x_indices_of_y):
        ctx.save_for_backward(x, a, b, w, given_x_indices_of_y_start, given_x_indices_of_y)
        y, _ = ops.logic_forward(x, a, b, w, ops.W_PROBS)
        return y

    @staticmethod
    def backward(ctx, grad_y):
        x, a, b, w, start, lst = ctx.saved_tensors
        grad_y = grad_y.contiguous()
        grad_w = grad_x = None
        if ctx.needs_input_grad[0]:
            plan = ops.build_backward_plan(a, b, start, lst)
            grad_x = ops.logic_backward_x(x, ops.logic_coefs(w, ops.W_PROBS), grad_y, start, plan, 1.0)
        if ctx.needs_input_grad[3]:
            grad_w = ops.logic_backward_w(x, a, b, grad_y, None, ops.W_PROBS)
        return grad_x, None, None, grad_w, None, None, None


class GroupSumFunction(torch.autograd.Function):
    """Float GroupSum on a 2-D CUDA tensor `[batch, n]`.  The output of a LogicLayer is a transposed view of a
    feature-major buffer, which the kernel reads as it is; any other layout is made feature-major first."""

    @staticmethod
    def forward(ctx, x, k, tau):
        ctx.k, ctx.tau, ctx.n = k, tau, x.shape[1]
        return ops.groupsum(x.transpose(0, 1).contiguous(), k, tau)

    @staticmethod
    def backward(ctx, grad_out):
        gx = ops.groupsum_backward(grad_out.contiguous(), ctx.n, ctx.tau)
        return gx.transpose(0, 1), None, None
