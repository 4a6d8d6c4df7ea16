"""CrossEntropyLoss for the class scores of a logic gate network, one kernel each way.

Same result as torch.nn.CrossEntropyLoss() (mean reduction, class-index targets, no weights, no label
smoothing) on a 2-D float32 CUDA input; anything else is handed to torch's implementation.
"""
import torch

from . import _native as N


class _CrossEntropyFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target):
        batch, k = logits.shape
        loss = torch.empty((), dtype=torch.float32, device=logits.device)
        probs = torch.empty_like(logits)
        with torch.cuda.device(logits.device):
            N.check(N.lib().dl_cross_entropy_f32(logits.data_ptr(), target.data_ptr(), loss.data_ptr(), probs.data_ptr(),
                                                 batch, k, N.stream_of(logits)))
        ctx.save_for_backward(probs, target)
        return loss

    @staticmethod
    def backward(ctx, grad_loss):
        probs, target = ctx.saved_tensors
        batch, k = probs.shape
        grad = torch.empty_like(probs)
        grad_loss = grad_loss.contiguous().to(torch.float32)
        with torch.cuda.device(probs.device):
            N.check(N.lib().dl_cross_entropy_backward_f32(probs.data_ptr(), target.data_ptr(), grad_loss.data_ptr(),
                                                          grad.data_ptr(), batch, k, N.stream_of(probs)))
        return grad, None


class _GroupSumCrossEntropyFunction(torch.autograd.Function):
    """cross_entropy(GroupSum(x), target) as ONE autograd node on the `[batch, n]` output of the last logic layer:
    forward = GroupSum kernel + loss kernel, backward = one kernel that writes the gradient of the layer's output
    straight from the softmax probabilities.  Same numbers as the two modules one after the other."""

    @staticmethod
    def forward(ctx, x, target, k, tau):
        from . import ops
        scores = ops.groupsum(x.transpose(0, 1).contiguous(), k, tau)
        batch = scores.shape[0]
        loss = torch.empty((), dtype=torch.float32, device=x.device)
        probs = torch.empty_like(scores)
        with torch.cuda.device(x.device):
            N.check(N.lib().dl_cross_entropy_f32(scores.data_ptr(), target.data_ptr(), loss.data_ptr(), probs.data_ptr(),
                                                 batch, k, N.stream_of(x)))
        ctx.save_for_backward(probs, target)
        ctx.k, ctx.tau, ctx.n = k, tau, x.shape[1]
        ctx.mark_non_differentiable(scores)
        ctx.set_materialize_grads(False)  # no zero-filled gradient for `scores`
        return loss, scores

    @staticmethod
    def backward(ctx, grad_loss, _grad_scores):
        if grad_loss is None:
            return None, None, None, None
        probs, target = ctx.saved_tensors
        batch = probs.shape[0]
        gx = torch.empty((ctx.n, batch), dtype=torch.float32, device=probs.device)
        grad_loss = grad_loss.contiguous().to(torch.float32)
        with torch.cuda.device(probs.device):
            N.check(N.lib().dl_groupsum_cross_entropy_backward_f32(probs.data_ptr(), target.data_ptr(), grad_loss.data_ptr(),
                                                                   gx.data_ptr(), ctx.n, batch, ctx.k, float(ctx.tau),
                                                                   N.stream_of(probs)))
        return gx.transpose(0, 1), None, None, None


def group_sum_cross_entropy(x, target, k, tau):
    """(loss, scores) of `CrossEntropyLoss()(GroupSum(k, tau)(x), target)` for a float32 CUDA `x` of shape
    `[batch, n]`; scores carries no gradient (use it for the accuracy)."""
    if not (x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and x.shape[0] > 0 and x.shape[1] % k == 0
            and target.dtype == torch.int64 and target.dim() == 1 and target.device == x.device):
        raise ValueError("group_sum_cross_entropy: needs a float32 CUDA [batch, n] input with n % k == 0 and int64 targets")
    return _GroupSumCrossEntropyFunction.apply(x, target.contiguous(), int(k), float(tau))


class CrossEntropyLoss(torch.nn.Module):
    """Drop-in for torch.nn.CrossEntropyLoss() with its default arguments."""

    def forward(self, input, target):
        if (input.is_cuda and input.dtype == torch.float32 and input.dim() == 2 and input.shape[0] > 0
                and target.dtype == torch.int64 and target.dim() == 1 and target.device == input.device):
            return _CrossEntropyFunction.apply(input.contiguous(), target.contiguous())
        return torch.nn.functional.cross_entropy(input, target)
