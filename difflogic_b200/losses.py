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


class CrossEntropyLoss(torch.nn.Module):
    """Drop-in for torch.nn.CrossEntropyLoss() with its default arguments."""

    def forward(self, input, target):
        if (input.is_cuda and input.dtype == torch.float32 and input.dim() == 2 and input.shape[0] > 0
                and target.dtype == torch.int64 and target.dim() == 1 and target.device == input.device):
            return _CrossEntropyFunction.apply(input.contiguous(), target.contiguous())
        return torch.nn.functional.cross_entropy(input, target)
