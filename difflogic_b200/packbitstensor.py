"""PackBitsTensor: a batch of boolean feature vectors packed along the batch dimension.

Drop-in for the reference class (difflogic/packbitstensor.py:6-41): `.t` is the packed tensor
`[features, ceil(batch / bit_count)]` of dtype int{bit_count}, `.pad_len` the number of unused
high bits in the last word, sample s being bit s % bit_count (LSB first) of word s // bit_count.
"""
import numpy as np
import torch

from . import ops


class PackBitsTensor:
    def __init__(self, t: torch.BoolTensor, bit_count=32, device='cuda'):
        assert len(t.shape) == 2, t.shape

        self.bit_count = bit_count
        self.device = device

        if device == 'cuda' or (isinstance(device, (str, torch.device)) and torch.device(device).type == 'cuda'):
            t = t.to(device)
            if t.dtype != torch.bool:
                t = t != 0
            # transpose and pack in one kernel, straight from the batch-major matrix
            self.t, self.pad_len = ops.packbits_batch_major(t.contiguous(), self.bit_count)
        else:
            raise NotImplementedError(device)

    @classmethod
    def from_packed(cls, words, pad_len, device='cuda'):
        """Wraps words that are already packed (e.g. a batch shard that was packed elsewhere)."""
        self = cls.__new__(cls)
        self.bit_count = ops.bits_of(words)
        self.device = device
        self.t = words
        self.pad_len = int(pad_len)
        return self

    def group_sum(self, k):
        assert torch.device(self.device).type == 'cuda', self.device
        return ops.groupbitsum(self.t, self.pad_len, k)

    def flatten(self, start_dim=0, end_dim=-1, **kwargs):
        """Returns the object itself so that torch.nn.Flatten passes it through; arguments are ignored."""
        return self

    def _row_repr(self, row):
        def word(v):
            return np.binary_repr(int(v), width=self.bit_count)[::-1]
        row = row.tolist()
        if len(row) <= 4:
            return ' '.join(word(v) for v in row)
        return '{} ... {}'.format(' '.join(word(v) for v in row[:3]), word(row[-1]))

    def __repr__(self):
        return '\n'.join(self._row_repr(row) for row in self.t.cpu())
